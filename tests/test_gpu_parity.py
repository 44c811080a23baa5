"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle on the same seeded
inputs, against the golden fixtures, and at the benchmark sizes through size-independent properties.

Tolerances of the fp16-in / fp32-accumulate paths: max-abs 2e-2 and relative Frobenius 1e-3 against
the fp32 oracle (oracle.MAX_ABS_TOL, oracle.REL_FRO_TOL). scatter_nd is bit-exact."""
import math

import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def assert_close(out, ref, max_abs=oracle.MAX_ABS_TOL, rel_fro=oracle.REL_FRO_TOL):
    ma, rf = oracle.max_abs_err(out, ref), oracle.rel_fro_err(out, ref)
    assert ma <= max_abs and rf <= rel_fro, f"max-abs {ma:.3g} (tol {max_abs}), rel-Frobenius {rf:.3g} (tol {rel_fro})"


# ------------------------------------------------------------------------------------------- GEMM
GEMM_SHAPES = [
        (16, 16, 16), (64, 128, 128),            # single-warp shapes of tests/cpp/cell/test_single_wmma.cu:190-195
        (128, 128, 64), (128, 256, 64),          # one tile of each kernel variant
        (32, 64, 32), (96, 48, 128), (128, 128, 128),  # shapes from tests/cpp/cell/test_gemm.cu:306-351
        (1, 8, 8), (129, 257, 72), (200, 300, 136), (1000, 24, 4104),  # ragged edges, K tail, many k-blocks
        (1024, 1024, 1024),                      # configuration C1
        (1024, 1024, 2048), (2048, 2048, 2048),
        (2304, 2304, 64), (2250, 2300, 136), (4100, 2310, 328),  # enough 256x256 tiles for the CTA-pair kernel, ragged edges
        (128, 19200, 256), (100, 19210, 264),    # one row tile, very wide: the lone 128x256 tiles
        (300, 520, 4096), (1536, 1536, 1536),    # few pair tiles with a long K loop
        (1290, 1410, 136),                       # lone 128x128 tiles with ragged edges
        (4000, 4090, 520),                       # 256 pair tiles on 74 pairs: three full waves and a partial one
        (640, 384, 576), (1000, 900, 1096), (130, 70, 520), (1024, 1024, 256), (128, 1024, 1024),  # single partial wave: odd K-block counts, ragged edges
    ]


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
def test_gemm_matches_oracle(cuda_ops, clean_status, m, n, k):
    a, b = oracle.gemm_inputs(m, n, k)
    c = torch.full((m, n), float("nan"), device=DEV)
    cuda_ops.gemm(a.to(DEV), b.to(DEV), c)
    # fp32 accumulation of exact fp16 products: far tighter than the stated tolerance
    assert_close(c, oracle.gemm(a, b), max_abs=2e-3, rel_fro=1e-5)


@pytest.mark.parametrize("tag", ["16", "64x128x128"])
def test_gemm_golden_ramp(cuda_ops, clean_status, golden_dir, tag):
    g = np.load(golden_dir / "gemm_ramp.npz")
    a, b, want = (torch.from_numpy(g[f"{x}_{tag}"]) for x in "abc")
    c = torch.empty(want.shape, device=DEV)
    cuda_ops.gemm(a.to(DEV), b.to(DEV), c)
    assert (c.cpu() - want).abs().max().item() < 1e-3  # the reference's own bound (test_single_wmma.cu:32)


def test_gemm_leading_dimensions_and_guard_bands(cuda_ops, clean_status):
    m, n, k = 200, 136, 264
    a_full, b_full = oracle.gemm_inputs(m, n, k + 24)
    a_dev, b_dev = a_full.to(DEV), b_full.to(DEV)
    c_store = torch.full((m + 2, n + 8), -7.0, device=DEV)
    c = c_store[1:m + 1, 4:n + 4]
    cuda_ops.gemm(a_dev[:, :k], b_dev[:, :k], c)
    assert_close(c, oracle.gemm(a_full[:, :k], b_full[:, :k]), max_abs=2e-3, rel_fro=1e-5)
    guard = c_store.clone()
    guard[1:m + 1, 4:n + 4] = -7.0
    assert (guard == -7.0).all(), "GEMM wrote outside its output"


@pytest.mark.parametrize("col_off,extra", [(4, 8), (1, 7)])
def test_gemm_guard_bands_aligned_and_unaligned_output(cuda_ops, clean_status, col_off, extra):
    """A single partial wave of tiles writing into a window of a larger buffer: with a 16-byte granular window the
    kernel stores through TMA, otherwise from registers; neither may touch the guard band around the window."""
    m, n, k = 900, 650, 1024
    a, b = oracle.gemm_inputs(m, n, k)
    c_store = torch.full((m + 2, n + extra), -7.0, device=DEV)
    c = c_store[1:m + 1, col_off:n + col_off]
    cuda_ops.gemm(a.to(DEV), b.to(DEV), c)
    assert_close(c, oracle.gemm(a, b), max_abs=2e-3, rel_fro=1e-5)
    guard = c_store.clone()
    guard[1:m + 1, col_off:n + col_off] = -7.0
    assert (guard == -7.0).all(), "GEMM wrote outside its output"


@pytest.mark.parametrize("max_sms", [140, 132, 64, 2])
def test_gemm_on_an_sm_budget_gives_the_same_result(cuda_ops, clean_status, max_sms):
    """tc_gemm_f16_f32_sms sizes the tile plan and the persistent grid for the budget; the result is the one of the
    unrestricted call (compared with the oracle, and bit for bit where both calls take the same tile shape)."""
    m, n, k = 4000, 4090, 520
    a, b = oracle.gemm_inputs(m, n, k)
    a_dev, b_dev = a.to(DEV), b.to(DEV)
    full, part = torch.empty(m, n, device=DEV), torch.full((m, n), float("nan"), device=DEV)
    cuda_ops.gemm(a_dev, b_dev, full)
    cuda_ops.gemm(a_dev, b_dev, part, max_sms=max_sms)
    assert_close(part, oracle.gemm(a, b), max_abs=2e-3, rel_fro=1e-5)
    assert torch.equal(part, full)   # every tile shape accumulates K in the same order


def test_gemm_linearity_at_sweep_size(cuda_ops, clean_status):
    """Size-independent property at 4096^3: (A1 + A2) B^T = A1 B^T + A2 B^T when the sum is exact in fp16."""
    n = 4096
    g = torch.Generator().manual_seed(oracle.SEED)
    a1 = (torch.randint(-8, 8, (n, n), generator=g).float() / 8).half().to(DEV)
    a2 = (torch.randint(-8, 8, (n, n), generator=g).float() / 8).half().to(DEV)
    b = (torch.randint(-8, 8, (n, n), generator=g).float() / 8).half().to(DEV)
    c1, c2, c12 = (torch.empty(n, n, device=DEV) for _ in range(3))
    cuda_ops.gemm(a1, b, c1)
    cuda_ops.gemm(a2, b, c2)
    cuda_ops.gemm(a1 + a2, b, c12)
    assert torch.equal(c12, c1 + c2)  # small dyadic values: every partial sum is exact in fp32
    rows = torch.arange(0, n, 257)
    assert torch.equal(c1[rows].cpu(), oracle.gemm(a1[rows].cpu(), b.cpu()))


def test_gemm_tall_pair_tiles_ragged_and_linear(cuda_ops, clean_status):
    """Operands far beyond L2 take the 512x256 pair tiles: ragged M and N with guard bands, sampled rows
    against the oracle (first, middle and last row tiles, both CTAs and both accumulator halves), and
    exact linearity over the whole result with small dyadic values."""
    m, n, k = 16384 + 328, 16384 - 56, 8192
    g = torch.Generator(device=DEV).manual_seed(oracle.SEED)
    mk = lambda r: (torch.randint(-8, 8, (r, k), generator=g, device=DEV, dtype=torch.int32).float() / 8).half()
    a1, a2, b = mk(m), mk(m), mk(n)
    store = torch.full((m + 2, n + 8), -7.0, device=DEV)
    c1 = store[1:m + 1, 4:n + 4]
    cuda_ops.gemm(a1, b, c1)
    rows = torch.cat([torch.arange(0, 512, 37), torch.arange(8192 + 100, 8192 + 612, 41), torch.arange(m - 330, m, 11)]).to(DEV)
    want = oracle.gemm(a1[rows].cpu(), b.cpu())
    assert torch.equal(c1[rows].cpu(), want)   # dyadic values: exact in fp32
    assert (store[0] == -7.0).all() and (store[-1] == -7.0).all()
    assert (store[:, :4] == -7.0).all() and (store[:, -4:] == -7.0).all()
    c2 = torch.empty(m, n, device=DEV)
    cuda_ops.gemm(a2, b, c2)
    c2 += c1
    cuda_ops.gemm(a1 + a2, b, c1)
    assert torch.equal(c1, c2)


@pytest.mark.parametrize("n", [8192, 16384])
def test_gemm_headline_sizes_on_the_benchmark_inputs(cuda_ops, clean_status, n):
    """The benchmark's own configuration: M = N = K = 8192 (the headline) and 16384, uniform[-1, 1) inputs from
    seed 1234 (oracle.gemm_inputs), through the C ABI. 96 rows are compared with the fp32 oracle: the first, a
    middle and the last 512-row pair tile, and in each both CTAs of the pair (rows 0-255 / 256-511 of the tile)
    and both 128-row accumulator halves of each CTA. The rest of the result is covered by a checksum: the column
    sums of C equal (sum of the rows of A) B^T, computed in float64 from the same inputs."""
    a, b = oracle.gemm_inputs(n, n, n)
    a_dev, b_dev = a.to(DEV), b.to(DEV)
    c = torch.full((n, n), float("nan"), device=DEV)
    cuda_ops.gemm(a_dev, b_dev, c)
    torch.cuda.synchronize()
    rows = []
    for tile0 in (0, (n // 1024) * 512, n - 512):
        for quarter in range(4):                       # CTA 0 half 0, CTA 0 half 1, CTA 1 half 0, CTA 1 half 1
            rows += [tile0 + quarter * 128 + r for r in (0, 17, 38, 59, 64, 85, 106, 127)]
    rows = torch.tensor(rows)
    assert rows.numel() == 96
    got = c[rows.to(DEV)].cpu()
    # The tensor core adds each K = 16 partial product into its fp32 accumulator with truncation, so the error grows
    # with the number of accumulation steps (K / 16): about 2e-3 at K = 8192 on entries of magnitude 30-150, twice that
    # at 16384. Bounds: half the stated max-abs tolerance of the path (2e-2) and a twentieth of its relative one (1e-3).
    assert_close(got, oracle.gemm(a[rows], b), max_abs=1e-2, rel_fro=5e-5)
    # checksum over every row: sum_i C[i, :] against (sum_i A[i, :]) B^T in float64
    col_sums = c.double().sum(dim=0).cpu()
    want = (a.double().sum(dim=0, keepdim=True) @ b.double().t()).view(-1)
    assert not torch.isnan(col_sums).any()
    assert (col_sums - want).abs().max().item() <= 2e-2 * math.sqrt(n)   # n entries whose errors have random signs


@pytest.mark.gpu
def test_gemm_launches_queued_back_to_back_keep_stream_order(cuda_ops, clean_status):
    """The GEMM kernels release the launch behind them early and start early themselves (programmatic stream
    serialization); memory effects must still follow stream order. The second GEMM writes its result over the
    first one's A operand, the third reads what the second wrote: neither may happen before its predecessor ends."""
    m, k = 2048, 2048
    a, b = oracle.gemm_inputs(m, 1024, k)
    a_dev, b_dev = a.to(DEV), b.to(DEV)
    c1 = torch.empty(m, 1024, device=DEV)
    a2, b2 = oracle.gemm_inputs(m, k // 2, 64, seed=5)
    a2_dev, b2_dev = a2.to(DEV), b2.to(DEV)
    c2_over_a = a_dev.view(torch.float32)            # [m, k / 2] fp32 on the bytes of A
    c3 = torch.empty(m, k // 2, device=DEV)
    for _ in range(3):
        a_dev.copy_(a)
        cuda_ops.gemm(a_dev, b_dev, c1)               # reads A ...
        cuda_ops.gemm(a2_dev, b2_dev, c2_over_a)      # ... which this one overwrites
        cuda_ops.gemm(a2_dev, b2_dev, c3)
        torch.cuda.synchronize()
        assert oracle.within_tolerance(c1, oracle.gemm(a, b))
        assert torch.equal(c2_over_a, c3)


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (200, 300, 136), (1024, 1024, 1024), (2250, 2300, 136)])
def test_gemm_bf16_inputs(cuda_ops, clean_status, m, n, k):
    """bf16 operands through the same kernels (all three tile variants): exact products, fp32 accumulation."""
    g = torch.Generator().manual_seed(oracle.SEED)
    a = (torch.rand(m, k, generator=g) * 2 - 1).bfloat16()
    b = (torch.rand(n, k, generator=g) * 2 - 1).bfloat16()
    c = torch.full((m, n), float("nan"), device=DEV)
    cuda_ops.gemm(a.to(DEV), b.to(DEV), c)
    assert_close(c, a.float() @ b.float().t(), max_abs=2e-3, rel_fro=1e-5)


# --------------------------------------------------------------------------------------- B2B GEMM
@pytest.mark.parametrize(
    "m,n,k,p,batch",
    [
        (16, 16, 16, 16, 1), (16, 32, 16, 32, 1), (32, 64, 32, 64, 1), (64, 64, 32, 64, 1),
        (256, 128, 64, 64, 1), (1024, 1024, 128, 128, 1), (16, 16, 16, 16, 2), (64, 256, 128, 128, 1),
        (2048, 1024, 128, 128, 1),                 # the shapes of examples/cpp/02_fused_two_gemms/fused_gemm.cu:212-259
        (2048, 2048, 128, 128, 1),                 # the shape the reference records as failing (:261-264)
        (200, 328, 48, 80, 3), (1000, 136, 128, 112, 2),  # ragged rows, inner tail, odd widths
    ],
)
def test_b2b_gemm_matches_oracle(cuda_ops, clean_status, m, n, k, p, batch):
    a, b, d = oracle.b2b_inputs(m, n, k, p, batch)
    e = torch.full((batch, m, p), float("nan"), device=DEV)
    cuda_ops.back2back_gemm(a.to(DEV), b.to(DEV), d.to(DEV), e)
    assert_close(e, oracle.back2back_gemm(a, b, d))


def test_b2b_gemm_configuration_c2(cuda_ops, clean_status):
    a, b, d = oracle.b2b_inputs(16384, 128, 128, 128, 1)
    e = torch.empty(16384, 128, device=DEV)
    cuda_ops.back2back_gemm(a[0].to(DEV), b[0].to(DEV), d[0].to(DEV), e)
    assert_close(e, oracle.back2back_gemm(a[0], b[0], d[0]))


# -------------------------------------------------------------------------------------- attention
@pytest.mark.parametrize("n", [64, 128, 256])
def test_flash_attention_fwd_reference_signature_and_golden(cuda_ops, clean_status, golden_dir, n):
    """The reference's op and wrapper conventions (pytiledcuda/__init__.py:17-36) on the reference's test
    inputs, against the output of the reference's own Python oracle; its tolerance is 8e-2 per element
    (tests/python/test_flash_attn.py:114), ours is the 2e-2 stated for this path."""
    g = np.load(golden_dir / f"flash_attn_ref_n{n}.npz")
    q, k_t, v, o_ref = (torch.from_numpy(g[x]) for x in ("q", "k_t", "v", "o"))
    m, k = q.shape
    p = v.shape[1]
    qd = q.to(DEV).flatten()
    kd = k_t.to(DEV).t().contiguous().flatten()   # the wrapper passes K as [n, k]
    vd = v.to(DEV).t().contiguous().flatten()     # and V as V^T [p, n]
    o = torch.full((m * p,), float("nan"), dtype=torch.float16, device=DEV)
    cuda_ops.flash_attention_fwd(qd, kd, vd, o, m, n, k, p)
    assert oracle.max_abs_err(o.view(m, p), o_ref) <= 2e-2
    direct, _ = oracle.flash_attention(q, k_t.t(), v, scale=1.0)
    assert_close(o.view(m, p), direct)


@pytest.mark.parametrize(
    "b,h,sq,skv,d,dv,vt",
    [
        (1, 1, 128, 128, 128, 128, False), (1, 1, 128, 128, 128, 128, True),
        (2, 3, 256, 384, 64, 64, False), (1, 2, 200, 328, 128, 128, False), (1, 2, 200, 328, 128, 128, True),
        (1, 1, 1, 8, 16, 16, False), (1, 2, 77, 1001, 80, 48, False), (1, 1, 130, 72, 32, 128, True),
        (2, 4, 1024, 1024, 128, 128, False),
        # more than one query tile against one, two and three half blocks of KV rows (the shortest pipelines of the two-tile kernel)
        (1, 2, 256, 64, 64, 64, False), (1, 1, 300, 40, 128, 128, False), (1, 2, 384, 128, 128, 128, False), (1, 1, 512, 192, 128, 128, False),
    ],
)
def test_flash_attn_matches_oracle(cuda_ops, clean_status, b, h, sq, skv, d, dv, vt):
    q, k, v = oracle.attention_inputs(b, h, sq, skv, d, dv)
    o = torch.full((b, h, sq, dv), float("nan"), dtype=torch.float16, device=DEV)
    lse = torch.empty(b, h, sq, device=DEV)
    vd = v.to(DEV).transpose(2, 3).contiguous() if vt else v.to(DEV)
    cuda_ops.flash_attn(q.to(DEV), k.to(DEV), vd, o, lse=lse, v_is_transposed=vt)
    ref, ref_lse = oracle.flash_attention(q, k, v)
    assert_close(o, ref)
    assert (lse.cpu() - ref_lse).abs().max().item() < 1e-3


@pytest.mark.parametrize(
    "b,h,sq,skv,d,dv",
    [
        (1, 1, 128, 128, 128, 128), (2, 3, 256, 256, 64, 64), (1, 2, 200, 328, 128, 128), (1, 2, 77, 1001, 80, 48),
        (1, 1, 1, 8, 16, 16), (1, 2, 640, 640, 128, 128), (1, 1, 300, 200, 64, 64), (2, 4, 1024, 1024, 128, 128),
        (1, 1, 2048, 2048, 128, 128),
    ],
)
def test_flash_attn_causal_matches_oracle(cuda_ops, clean_status, b, h, sq, skv, d, dv):
    """Bottom-right aligned causal mask, ragged sizes included; with seq_q > seq_kv the first rows see nothing
    and come back as zeros with lse = -inf."""
    q, k, v = oracle.attention_inputs(b, h, sq, skv, d, dv)
    o = torch.full((b, h, sq, dv), float("nan"), dtype=torch.float16, device=DEV)
    lse = torch.empty(b, h, sq, device=DEV)
    cuda_ops.flash_attn(q.to(DEV), k.to(DEV), v.to(DEV), o, lse=lse, causal=True)
    ref, ref_lse = oracle.flash_attention(q, k, v, causal=True)
    assert_close(o, ref)
    seen = torch.isfinite(ref_lse)
    assert (lse.cpu()[seen] - ref_lse[seen]).abs().max().item() < 1e-3
    assert torch.isinf(lse.cpu()[~seen]).all()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("b,h,sq,skv,d,dv", [(2, 3, 256, 384, 64, 64), (1, 5, 100, 100, 128, 128), (2, 8, 1024, 1024, 128, 128)])
def test_flash_attn_seq_major_operands(cuda_ops, clean_status, causal, b, h, sq, skv, d, dv):
    """[batch, seq, heads, dim] operands give the same result as the head-major layout."""
    q, k, v = oracle.attention_inputs(b, h, sq, skv, d, dv)
    to_sm = lambda t: t.to(DEV).transpose(1, 2).contiguous()
    o = torch.full((b, sq, h, dv), float("nan"), dtype=torch.float16, device=DEV)
    lse = torch.empty(b, h, sq, device=DEV)
    cuda_ops.flash_attn(to_sm(q), to_sm(k), to_sm(v), o, lse=lse, causal=causal, seq_major=True)
    ref, ref_lse = oracle.flash_attention(q, k, v, causal=causal)
    assert_close(o.transpose(1, 2), ref)
    assert (lse.cpu() - ref_lse).abs().max().item() < 1e-3
    o2 = torch.empty(b, h, sq, dv, dtype=torch.float16, device=DEV)
    cuda_ops.flash_attn(q.to(DEV), k.to(DEV), v.to(DEV), o2, causal=causal)
    if sq > 128 or causal:   # same kernel, same arithmetic: bit-identical
        assert torch.equal(o.transpose(1, 2), o2)


@pytest.mark.parametrize(
    "b,h,sq,skv,d,dv,vt,seq_major",
    [
        (4, 40, 512, 320, 64, 64, False, False),     # 320 CTAs on 148 SMs, an odd number of half blocks per CTA
        (2, 80, 456, 1000, 128, 128, False, False),  # ragged query tail (second tile partly outside) and ragged KV tail
        (3, 50, 512, 256, 128, 128, True, False),    # V given transposed
        (2, 96, 256, 128, 64, 128, False, True),     # one query block per head, sequence-major operands, two half blocks
        (1, 160, 256, 64, 128, 128, False, False),   # a single half block per CTA
    ],
)
def test_flash_attn_more_ctas_than_sms_matches_oracle(cuda_ops, clean_status, b, h, sq, skv, d, dv, vt, seq_major):
    """Non-causal attention with more (batch x head, query block) CTAs than SMs, so that SMs take several CTAs in
    turn: odd and single half-block counts, ragged query and KV tails, transposed V, sequence-major operands. Output
    and LSE of every (batch, head) against the oracle."""
    q, k, v = oracle.attention_inputs(b, h, sq, skv, d, dv)
    lse = torch.empty(b, h, sq, device=DEV)
    ref, ref_lse = oracle.flash_attention(q, k, v)
    if seq_major:
        to_sm = lambda t: t.to(DEV).transpose(1, 2).contiguous()
        o = torch.full((b, sq, h, dv), float("nan"), dtype=torch.float16, device=DEV)
        cuda_ops.flash_attn(to_sm(q), to_sm(k), to_sm(v), o, lse=lse, seq_major=True)
        o = o.transpose(1, 2)
    else:
        o = torch.full((b, h, sq, dv), float("nan"), dtype=torch.float16, device=DEV)
        vd = v.to(DEV).transpose(2, 3).contiguous() if vt else v.to(DEV)
        cuda_ops.flash_attn(q.to(DEV), k.to(DEV), vd, o, lse=lse, v_is_transposed=vt)
    assert_close(o, ref)
    assert (lse.cpu() - ref_lse).abs().max().item() < 1e-3


def test_flash_attn_ex_rejects_bad_combinations(cuda_ops, clean_status):
    q = torch.zeros(1, 64, 2, 64, dtype=torch.float16, device=DEV)
    with pytest.raises(ValueError):
        cuda_ops.flash_attn(q, q, q, torch.empty_like(q), seq_major=True, v_is_transposed=True)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("sq,skv", [(256, 104), (384, 200), (128, 72)])
def test_flash_attn_with_a_zero_scale_averages_the_visible_rows(cuda_ops, clean_status, causal, sq, skv):
    """scale == 0 gives every visible KV row the same weight, also where columns are masked (a ragged last half block,
    the causal diagonal): masking is applied after scaling."""
    torch.manual_seed(5)
    q = torch.randn(1, 2, sq, 64, device=DEV).half()
    k = torch.randn(1, 2, skv, 64, device=DEV).half()
    v = torch.randn(1, 2, skv, 64, device=DEV).half()
    o = torch.full((1, 2, sq, 64), float("nan"), dtype=torch.float16, device=DEV)
    cuda_ops.flash_attn(q, k, v, o, causal=causal, scale=0.0)
    vf = v.float().cpu()
    want = torch.zeros(1, 2, sq, 64)
    for i in range(sq):
        visible = min(skv, i + (skv - sq) + 1) if causal else skv
        if visible > 0:
            want[:, :, i] = vf[:, :, :visible].mean(dim=2)
    assert torch.allclose(o.float().cpu(), want, atol=2e-3, rtol=2e-3)


def test_flash_attn_large_scores_need_rescaling(cuda_ops, clean_status):
    """Rows whose maximum grows block after block: exercises the deferred rescale of the accumulator."""
    b, h, s, d = 1, 2, 1024, 64
    q, k, v = oracle.attention_inputs(b, h, s, s, d)
    ramp = torch.linspace(0.2, 3.0, s).view(1, 1, s, 1)
    k = (k.float() * ramp).half()
    o = torch.empty(b, h, s, d, dtype=torch.float16, device=DEV)
    cuda_ops.flash_attn(q.to(DEV), k.to(DEV), v.to(DEV), o, scale=1.0)
    ref, _ = oracle.flash_attention(q, k, v, scale=1.0)
    assert_close(o, ref)


def test_flash_attn_configuration_c3_properties(cuda_ops, clean_status):
    """Full size of configuration C3 (batch 16, heads 32, seq 4096, dim 128). The fp32 CPU oracle checks
    sampled (batch, head) pairs; two properties cover the rest: with V = 1 every output is 1, and a
    permutation of the KV rows leaves the output unchanged up to rounding."""
    b, h, s, d = 16, 32, 4096, 128
    g = torch.Generator(device=DEV).manual_seed(oracle.SEED)
    q = torch.randn(b, h, s, d, generator=g, device=DEV, dtype=torch.float16)
    k = torch.randn(b, h, s, d, generator=g, device=DEV, dtype=torch.float16)
    v = torch.randn(b, h, s, d, generator=g, device=DEV, dtype=torch.float16)
    o = torch.empty_like(q)
    cuda_ops.flash_attn(q, k, v, o)
    for bi, hi in [(0, 0), (7, 13), (15, 31)]:
        ref, _ = oracle.flash_attention(q[bi, hi].cpu(), k[bi, hi].cpu(), v[bi, hi].cpu())
        assert_close(o[bi, hi], ref)
    perm = torch.randperm(s, generator=torch.Generator().manual_seed(1)).to(DEV)
    o2 = torch.empty_like(q)
    cuda_ops.flash_attn(q, k[:, :, perm].contiguous(), v[:, :, perm].contiguous(), o2)
    assert (o.float() - o2.float()).abs().max().item() <= 4e-3
    v.fill_(1.0)
    cuda_ops.flash_attn(q, k, v, o)
    assert (o.float() - 1.0).abs().max().item() <= 2e-3


# ------------------------------------------------------------------------------------------- LSTM
def test_lstm_cell_golden_torch(cuda_ops, clean_status, golden_dir):
    g = np.load(golden_dir / "lstm_cell_torch.npz")
    t = {k: torch.from_numpy(g[k]).to(DEV) for k in g.files}
    # golden batch is 24 rows of 40 inputs: both within the kernel's multiples (8, 16)
    h1 = torch.empty_like(t["h"])
    c1 = torch.empty_like(t["c"])
    cuda_ops.lstm_cell(t["w"], t["u"], t["bias"], t["x"], t["h"], t["c"], h1, c1)
    assert_close(h1, t["h1"])
    assert_close(c1, t["c1"])


@pytest.mark.parametrize("batch,inp,hidden,bias", [(128, 64, 16, True), (100, 72, 48, True), (256, 1024, 1024, False),
                                                    (256, 256, 4096, True), (1, 8, 16, False),
                                                    # odd numbers of 64-wide K blocks (ring stages hold two): 3 + 7 with
                                                    # 16-unit tiles, 2 + 75 with 32-unit tiles
                                                    (200, 192, 448, True), (64, 128, 4800, False)])
def test_lstm_cell_matches_oracle(cuda_ops, clean_status, batch, inp, hidden, bias):
    w, u, b, x, _, _ = oracle.lstm_inputs(1, batch, inp, hidden, with_bias=bias)
    g = torch.Generator().manual_seed(7)
    h = (torch.randn(batch, hidden, generator=g) * 0.5).half()
    c = torch.randn(batch, hidden, generator=g)
    h1 = torch.full((batch, hidden), float("nan"), dtype=torch.float16, device=DEV)
    c1 = torch.full((batch, hidden), float("nan"), device=DEV)
    cuda_ops.lstm_cell(w.to(DEV), u.to(DEV), None if b is None else b.to(DEV), x[0].to(DEV), h.to(DEV), c.to(DEV), h1, c1)
    rh, rc = oracle.lstm_cell(w, u, b, x[0], h, c)
    assert_close(h1, rh)
    assert_close(c1, rc)


def test_lstm_chain_configuration_c4(cuda_ops, clean_status):
    steps, batch, inp, hidden = 64, 256, 1024, 1024
    w, u, b, x, h0, c0 = oracle.lstm_inputs(steps, batch, inp, hidden)
    h_all = torch.empty(steps, batch, hidden, dtype=torch.float16, device=DEV)
    c_t = torch.empty(batch, hidden, device=DEV)
    cuda_ops.lstm_chain(w.to(DEV), u.to(DEV), None, x.to(DEV), h0.to(DEV), c0.to(DEV), h_all, c_t)
    rh, rc = oracle.lstm_chain(w, u, b, x, h0, c0)
    assert_close(h_all, rh)
    assert_close(c_t, rc)
    # the chain equals the cell applied step by step (same kernel, same bits)
    h_prev, c_prev = h0.to(DEV), c0.to(DEV)
    for t in range(3):
        h1 = torch.empty_like(h_prev)
        c1 = torch.empty_like(c_prev)
        cuda_ops.lstm_cell(w.to(DEV), u.to(DEV), None, x[t].to(DEV), h_prev, c_prev, h1, c1)
        assert torch.equal(h1, h_all[t])
        h_prev, c_prev = h1, c1


@pytest.mark.parametrize("steps,batch,inp,hidden,bias", [(5, 100, 72, 48, True), (64, 256, 1024, 1024, False),
                                                          (3, 130, 136, 448, True)])
def test_lstm_chain_with_workspace_matches_oracle_and_plain_chain(cuda_ops, clean_status, steps, batch, inp, hidden, bias):
    """The chain that hoists x W^T of all steps into one GEMM (caller-provided scratch) against the oracle and
    against the chain without scratch."""
    w, u, b, x, h0, c0 = oracle.lstm_inputs(steps, batch, inp, hidden, with_bias=bias)
    dev = [t.to(DEV) if t is not None else None for t in (w, u, b, x, h0, c0)]
    h_ws = torch.empty(steps, batch, hidden, dtype=torch.float16, device=DEV)
    c_ws = torch.empty(batch, hidden, device=DEV)
    nbytes = cuda_ops.lstm_chain_workspace_bytes(steps, batch, hidden)
    assert nbytes == steps * batch * 4 * hidden * 4
    ws = torch.empty(nbytes // 4, device=DEV)
    cuda_ops.lstm_chain(*dev, h_ws, c_ws, workspace=ws)
    rh, rc = oracle.lstm_chain(w, u, b, x, h0, c0)
    assert_close(h_ws, rh)
    assert_close(c_ws, rc)
    h_plain = torch.empty_like(h_ws)
    c_plain = torch.empty_like(c_ws)
    cuda_ops.lstm_chain(*dev, h_plain, c_plain)
    assert_close(h_ws, h_plain, max_abs=2e-3, rel_fro=2e-4)
    with pytest.raises(Exception, match="workspace"):
        cuda_ops.lstm_chain(*dev, h_ws, c_ws, workspace=ws[: ws.numel() // 2])


# ------------------------------------------------------------------------------------- scatter_nd
def test_scatter_nd_reference_test_case(cuda_ops, clean_status, golden_dir):
    """tests/python/test_scatter_nd.py:22-54: data [7,8,9,10] fp32, five (i, j) pairs, 90-element slices."""
    g = np.load(golden_dir / "scatter_nd_ref.npz")
    data = torch.from_numpy(g["data"]).to(DEV)
    cuda_ops.scatter_nd(data, torch.from_numpy(g["indices"]).to(DEV), torch.from_numpy(g["updates"]).to(DEV))
    assert data.cpu().numpy().tobytes() == g["out"].tobytes()
    data2 = torch.from_numpy(g["data2"]).to(DEV)
    cuda_ops.scatter_nd(data2, torch.from_numpy(g["indices2"]).to(DEV), torch.from_numpy(g["updates2"]).to(DEV))
    assert data2.cpu().numpy().tobytes() == g["out2"].tobytes()


@pytest.mark.parametrize("index_dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("rows,width,n,dtype", [(1000, 8, 300, torch.float16), (4096, 3, 4096, torch.float16),
                                                 (257, 5, 100, torch.float32), (64, 1, 64, torch.int8),
                                                 (1 << 20, 8, 1 << 18, torch.float16)])
def test_scatter_nd_rows_bit_exact(cuda_ops, clean_status, rows, width, n, dtype, index_dtype):
    g = torch.Generator().manual_seed(oracle.SEED)
    table = torch.randint(-100, 100, (rows, width), generator=g).to(dtype)
    idx = torch.randperm(rows, generator=g)[:n].to(index_dtype).view(n, 1)
    upd = torch.randint(-100, 100, (n, width), generator=g).to(dtype)
    dev_table = table.to(DEV)
    cuda_ops.scatter_nd(dev_table, idx.to(DEV), upd.to(DEV))
    want = oracle.scatter_nd(table.numpy(), idx.numpy(), upd.numpy())
    assert dev_table.cpu().numpy().tobytes() == want.tobytes()


def test_scatter_nd_rank3_tuples_and_empty(cuda_ops, clean_status):
    g = torch.Generator().manual_seed(3)
    data = torch.randn(5, 6, 7, 4, generator=g)
    flat = torch.randperm(5 * 6 * 7, generator=g)[:50]
    idx = torch.stack([flat // 42, (flat // 7) % 6, flat % 7], dim=1)
    upd = torch.randn(50, 4, generator=g)
    dev = data.to(DEV)
    cuda_ops.scatter_nd(dev, idx.to(DEV), upd.to(DEV))
    assert dev.cpu().numpy().tobytes() == oracle.scatter_nd(data.numpy(), idx.numpy(), upd.numpy()).tobytes()
    before = dev.clone()
    cuda_ops.scatter_nd(dev, torch.zeros(0, 3, dtype=torch.int64, device=DEV), torch.zeros(0, 4, device=DEV))
    assert torch.equal(dev, before)


def test_scatter_nd_out_of_range_is_skipped_and_reported(cuda_ops):
    from tiledcuda_b200 import _lib

    _lib.device_status()
    data = torch.zeros(16, 8, dtype=torch.float16, device=DEV)
    idx = torch.tensor([[3], [16], [-1], [5]], dtype=torch.int32, device=DEV)
    upd = torch.ones(4, 8, dtype=torch.float16, device=DEV)
    cuda_ops.scatter_nd(data, idx, upd)
    assert _lib.device_status() == 16  # kDevIndexOutOfRange
    assert data.sum().item() == 16.0 and data[3].sum().item() == 8.0 and data[5].sum().item() == 8.0
    assert _lib.device_status() == 0


def test_scatter_nd_configuration_c5_checksums(cuda_ops, clean_status):
    """Full size of configuration C5: 2^24 unique rows into a [2^26, 8] fp16 table. Checked bit-exact against the
    numpy oracle on the whole table."""
    rows, width, n = 1 << 26, 8, 1 << 24
    table, idx, upd = oracle.scatter_inputs(rows, width, n)
    dev = table.to(DEV)
    cuda_ops.scatter_nd(dev, idx.to(DEV), upd.to(DEV))
    want = torch.from_numpy(oracle.scatter_nd(table.numpy(), idx.numpy(), upd.numpy()))
    assert torch.equal(dev.cpu().view(torch.int16), want.view(torch.int16))
    # idempotence: applying the same updates again changes nothing
    again = dev.clone()
    cuda_ops.scatter_nd(again, idx.to(DEV), upd.to(DEV))
    assert torch.equal(again.view(torch.int16), dev.view(torch.int16))


@pytest.mark.parametrize("index_dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("rows,width,n,dtype", [(1000, 8, 3000, torch.float16), (4096, 3, 4096, torch.float16),
                                                 (257, 5, 1000, torch.float32), (257, 4, 1000, torch.float32),
                                                 (64, 1, 640, torch.int32), (500, 4, 2000, torch.int32),
                                                 (100, 2, 700, torch.float64), (100, 3, 700, torch.float64),
                                                 (1 << 18, 8, 1 << 20, torch.float32)])
def test_scatter_nd_add_with_repeated_rows(cuda_ops, clean_status, rows, width, n, dtype, index_dtype):
    """Accumulation with repeated index tuples. Small integer values keep every partial sum exactly
    representable in each type, so the unspecified order of the additions cannot show and the comparison is
    bit-exact."""
    g = torch.Generator().manual_seed(oracle.SEED)
    table = torch.randint(-8, 8, (rows, width), generator=g).to(dtype)
    idx = torch.randint(0, rows, (n, 1), generator=g).to(index_dtype)
    upd = torch.randint(-4, 4, (n, width), generator=g).to(dtype)
    dev_table = table.to(DEV)
    cuda_ops.scatter_nd_add(dev_table, idx.to(DEV), upd.to(DEV))
    want = oracle.scatter_nd_add(table.numpy(), idx.numpy(), upd.numpy())
    assert dev_table.cpu().numpy().tobytes() == want.tobytes()


def test_scatter_nd_add_reference_shape_and_linearity(cuda_ops, clean_status, golden_dir):
    """The reference test's inputs (tests/python/test_scatter_nd.py:22-54; one tuple occurs twice) in
    accumulating mode on a zero table: equal to the accumulating oracle (two addends commute, so bit-exact);
    applying the updates twice doubles the table up to rounding; out-of-range tuples are skipped and reported."""
    from tiledcuda_b200 import _lib

    g = np.load(golden_dir / "scatter_nd_ref.npz")
    idx = torch.from_numpy(g["indices"]).to(DEV)
    upd = torch.from_numpy(g["updates"]).to(DEV)
    zero = torch.zeros_like(torch.from_numpy(g["data"])).to(DEV)
    cuda_ops.scatter_nd_add(zero, idx, upd)
    want = oracle.scatter_nd_add(np.zeros_like(g["data"]), g["indices"], g["updates"])
    assert zero.cpu().numpy().tobytes() == want.tobytes()
    cuda_ops.scatter_nd_add(zero, idx, upd)
    np.testing.assert_allclose(zero.cpu().numpy(), 2 * want, rtol=1e-6, atol=1e-6)
    data = torch.zeros(16, 8, dtype=torch.float32, device=DEV)
    bad = torch.tensor([[3], [16], [-1], [3]], dtype=torch.int32, device=DEV)
    cuda_ops.scatter_nd_add(data, bad, torch.ones(4, 8, device=DEV))
    assert _lib.device_status() == 16
    assert data.sum().item() == 16.0 and data[3].sum().item() == 16.0
    with pytest.raises(TypeError):
        cuda_ops.scatter_nd_add(torch.zeros(4, 4, dtype=torch.int8, device=DEV), bad[:1], torch.zeros(1, 4, dtype=torch.int8, device=DEV))


# ---------------------------------------------------------------------------------- error behaviour
def test_unsupported_shapes_raise(cuda_ops):
    from tiledcuda_b200._lib import TiledCudaError

    a = torch.zeros(128, 60, dtype=torch.float16, device=DEV)
    with pytest.raises(TiledCudaError, match="multiple of 8"):
        cuda_ops.gemm(a, a, torch.zeros(128, 128, device=DEV))
    q = torch.zeros(1, 1, 128, 256, dtype=torch.float16, device=DEV)
    with pytest.raises(TiledCudaError, match=r"\[16,128\]"):
        cuda_ops.flash_attn(q, q, q, torch.zeros_like(q))
    with pytest.raises(TypeError):
        cuda_ops.gemm(a.float(), a, torch.zeros(128, 128, device=DEV))


# ------------------------------------------------------------------------------- host-buffer GEMM
@pytest.mark.parametrize("m,n,k", [(512, 384, 256), (2304, 2048, 512), (8192, 2560, 264), (1000, 4104, 72)])
def test_gemm_host_pipelined_matches_oracle(cuda_ops, clean_status, m, n, k):
    """The host-operand entry point (uploads, block products and downloads overlapped) against the oracle,
    with guard values around the host result."""
    a, b = oracle.gemm_inputs(m, n, k)
    ha, hb = a.pin_memory(), b.pin_memory()
    hc = torch.full((m, n), float("nan"), dtype=torch.float32).pin_memory()
    ws = torch.empty(cuda_ops.gemm_host_workspace_bytes(m, n, k), dtype=torch.uint8, device=DEV)
    cuda_ops.gemm_host(ha, hb, hc, ws)
    torch.cuda.synchronize()
    assert_close(hc, oracle.gemm(a, b), max_abs=2e-3, rel_fro=1e-5)
    cuda_ops.gemm_host(ha, hb, hc, ws)   # a second call reuses the internal streams and events
    torch.cuda.synchronize()
    assert_close(hc, oracle.gemm(a, b), max_abs=2e-3, rel_fro=1e-5)
