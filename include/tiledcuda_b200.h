/* C ABI of the B200-native TiledCUDA tile-kernel path (libtiledcuda_b200.so).
 *
 * Every entry point takes raw device pointers, plain integer sizes and a CUDA stream, launches on
 * that stream and returns without synchronising. Return value: 0 on success, a negative tc_status
 * otherwise; tc_last_error() then holds a message for the calling thread. Nothing here allocates on
 * the hot path except the one-time per-device status word, and nothing calls exit().
 *
 * Each declaration cites the interface of the TiledCUDA reference that it stands in for.
 */
#ifndef TILEDCUDA_B200_H_
#define TILEDCUDA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* tc_stream_t; /* a cudaStream_t; NULL is the default stream */

enum tc_status {
    TC_OK = 0,
    TC_ERR_BAD_ARG = -1,     /* null pointer, bad shape, misaligned pointer or stride */
    TC_ERR_UNSUPPORTED = -2, /* shape or device outside what the kernels cover (needs sm_100) */
    TC_ERR_CUDA = -3,        /* a CUDA runtime / driver call failed; message has the CUDA error */
    TC_ERR_DEVICE = -4       /* a kernel recorded an error in the device status word */
};

/* Message of the last failing call made by this thread ("" if none). */
const char* tc_last_error(void);

/* ABI version of this library (major*1000 + minor). */
int tc_version(void);

/* Reads and clears the status word that kernels write when a bounded wait ran out or an index was
 * out of range. Synchronises the current device. *code receives 0 when all launches were clean.
 * Replaces the reference's CudaCheck -> exit(EXIT_FAILURE) (include/cuda_utils.hpp:20-26). */
int tc_device_status(int* code);

/* C[M,N] (fp32, row-major, leading dimension ldc) = A[M,K] (fp16, row-major, lda) * B, where B is
 * column-major [K,N], i.e. stored as [N,K] row-major with leading dimension ldb.
 * Needs K % 8 == 0, lda % 8 == 0, ldb % 8 == 0 and 16-byte aligned A and B.
 * Replaces the reference's GEMM kernels `gemm` (examples/cpp/01_gemm/02_gemm_all_mem/gemm.hpp:92-155)
 * and `simple_gemm` (examples/cpp/01_gemm/01_gemm_global_reg/gemm.hpp:59-92), and follows the C-ABI
 * precedent `kernel_entry(__half*, __half*, float*)` (examples/python/gemm/entry.py:56-68). */
int tc_gemm_f16_f32(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                    int64_t ldb, int64_t ldc, tc_stream_t stream);

/* tc_gemm_f16_f32 on at most max_sms streaming multiprocessors (0 = all of them): the tile plan and the persistent
 * grid are sized for that budget and the other SMs stay free for kernels that run beside the GEMM, e.g. the
 * collective that assembles finished row blocks of C on the other GPUs while later blocks are computed. The
 * reference is single-GPU and sizes its grid by the problem alone (examples/cpp/01_gemm/02_gemm_all_mem/main.cu:67-71);
 * it has no counterpart there. */
int tc_gemm_f16_f32_sms(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                        int64_t ldb, int64_t ldc, int max_sms, tc_stream_t stream);

/* The same GEMM with bf16 A and B (fp32 accumulate and output). The reference is fp16-only
 * (include/cell/compute/gemm.hpp:26-29 static_asserts); it has no counterpart there. */
int tc_gemm_bf16_f32(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                     int64_t ldb, int64_t ldc, tc_stream_t stream);

/* Which tile shape tc_gemm_f16_f32 / tc_gemm_bf16_f32 run a problem with on a device of sm_count SMs (148 on
 * B200): a pure function of its arguments, usable without a GPU. Returns one of TC_GEMM_TILE_* (or a negative
 * status). It stands where the reference picks tile shapes by compiling and timing candidate kernels at run time
 * (examples/python/gemm/main.py:37-70 with compile.py:83-127); here the table is fixed ahead of time from
 * measurements. */
enum {
    TC_GEMM_TILE_128x128 = 0,       /* lone CTA, 128x128, six K blocks of 64 in flight */
    TC_GEMM_TILE_128x256 = 1,       /* lone CTA, 128x256x64, four stages */
    TC_GEMM_TILE_PAIR_256x256 = 2,  /* CTA pair, tcgen05.mma.cta_group::2, double-buffered accumulators */
    TC_GEMM_TILE_PAIR_512x256 = 3,  /* CTA pair, two accumulator halves per CTA */
    TC_GEMM_TILE_128x64 = 4         /* lone CTA, 128x64: problems whose 128x128 tiles would leave half the SMs idle */
};
int tc_gemm_tile_plan(int64_t M, int64_t N, int64_t K, int sm_count);

/* The same GEMM with HOST operands and result (contiguous: lda = ldb = K, ldc = N), for callers whose data
 * lives in host memory, as the reference's Python examples' does before `.cuda()`
 * (examples/python/gemm/main.py:47-52). Uploads, products and downloads are pipelined block by block over
 * both directions of the host link on internal streams; on return everything is queued and `stream` is
 * ordered after the last download (synchronise it before reading hC). d_workspace is caller-owned device
 * memory of tc_gemm_host_workspace_bytes(M, N, K) bytes, 256-byte aligned; host buffers should be pinned.
 * Calls on one device must not overlap (they share the internal streams' events). */
int64_t tc_gemm_host_workspace_bytes(int64_t M, int64_t N, int64_t K);
int tc_gemm_f16_f32_host(const void* hA, const void* hB, void* hC, int64_t M, int64_t N, int64_t K, void* d_workspace,
                         int64_t workspace_bytes, tc_stream_t stream);

/* E[b] (fp32 [M,P]) = fp16(A[b] * B[b]) * D[b] for b in [0,batch): A fp16 [M,K] row-major; B
 * column-major [K,N] stored as [N,K]; D column-major [N,P] stored as [P,N]. The intermediate A*B is
 * accumulated in fp32, rounded to fp16 and never leaves the chip.
 * Needs K % 16 == 0, K <= 128, P % 16 == 0, P <= 128, N % 8 == 0.
 * Replaces `KeFusedGemm` (examples/cpp/02_fused_two_gemms/fused_gemm.hpp:98-181). */
int tc_b2b_gemm_f16(const void* A, const void* B, const void* D, void* E, int64_t M, int64_t N, int64_t K,
                    int64_t P, int64_t batch, tc_stream_t stream);

/* O = softmax(scale * Q K^T) V per (batch, head), non-causal. Q [batch,heads,seq_q,head_dim],
 * K [batch,heads,seq_kv,head_dim], O [batch,heads,seq_q,head_dim_v], all fp16 and contiguous;
 * V is [batch,heads,seq_kv,head_dim_v] when v_is_transposed == 0, or V^T
 * [batch,heads,head_dim_v,seq_kv] (the layout the reference's Python wrapper produces) otherwise.
 * lse (fp32 [batch,heads,seq_q], natural log of the softmax denominator) may be NULL.
 * Softmax statistics are fp32. Needs head_dim, head_dim_v multiples of 16 and <= 128; seq_kv % 8 == 0 when V is
 * transposed (rows of V^T are 16-byte granular); scale finite (zero weighs every KV row the same).
 * Replaces `flash_attention` / `run_flash_attention` / `custom_flash_attention_op`
 * (src/kernels/flash_attn.cu:134-312, 314-422, 424-456); the reference fixes scale = 1. */
int tc_flash_attn_fwd_f16(const void* Q, const void* K, const void* V, void* O, float* lse, int64_t batch,
                          int64_t heads, int64_t seq_q, int64_t seq_kv, int64_t head_dim, int64_t head_dim_v,
                          float scale, int v_is_transposed, tc_stream_t stream);

/* The same attention with two options the reference's kernel does not have (no counterpart in the
 * reference: its flash_attention, src/kernels/flash_attn.cu:134-312, is non-causal over
 * [batch*heads, seq, dim] operands). causal != 0: query row i sees KV rows j <= i + (seq_kv - seq_q),
 * i.e. the mask is aligned to the bottom-right corner; KV blocks above the diagonal are skipped, a row
 * that sees no KV row yields zeros and lse = -inf. seq_major != 0: Q, K, V and O
 * are [batch, seq, heads, dim] (heads interleaved per token, as a fused QKV projection leaves them)
 * instead of [batch, heads, seq, dim]; not together with a transposed V. lse stays [batch, heads, seq_q]. */
int tc_flash_attn_fwd_ex_f16(const void* Q, const void* K, const void* V, void* O, float* lse, int64_t batch,
                             int64_t heads, int64_t seq_q, int64_t seq_kv, int64_t head_dim, int64_t head_dim_v,
                             float scale, int v_is_transposed, int causal, int seq_major, tc_stream_t stream);

/* One LSTM cell step, gate order (i, f, g, o) as torch.nn.LSTMCell:
 *   gates = x W^T + h_prev U^T + bias;  c_out = sigmoid(f) c_prev + sigmoid(i) tanh(g);
 *   h_out = sigmoid(o) tanh(c_out).
 * W fp16 [4*hidden, input], U fp16 [4*hidden, hidden], bias fp32 [4*hidden] or NULL, x fp16
 * [batch,input], h_prev / h_out fp16 [batch,hidden], c_prev / c_out fp32 [batch,hidden].
 * h_out must not alias h_prev; c_out may alias c_prev (updated in place). Needs input % 8 == 0, hidden % 16 == 0.
 * The reference snapshot names this op (Makefile:3, test_lstm_cell) but ships no code for it. */
int tc_lstm_cell_f16(const void* W, const void* U, const float* bias, const void* x, const void* h_prev,
                     const float* c_prev, void* h_out, float* c_out, int64_t batch, int64_t input,
                     int64_t hidden, tc_stream_t stream);

/* `steps` chained LSTM cells (the recurrence of tc_lstm_cell_f16, one launch per step on `stream`):
 * x fp16 [steps,batch,input]; h0 fp16 [batch,hidden]; c0 fp32 [batch,hidden]; h_all fp16
 * [steps,batch,hidden] receives every h_t (its last slab is h_T); c_out fp32 [batch,hidden] receives
 * c_T (it is also the running cell state, updated in place after the first step). c_out may alias c0.
 * The cell state stays fp32 across steps; h_t is rounded to fp16 where it feeds the next step.
 * Like the cell, it has no code in the reference snapshot (Makefile:3 only names test_lstm_cell). */
int tc_lstm_chain_f16(const void* W, const void* U, const float* bias, const void* x, const void* h0,
                      const float* c0, void* h_all, float* c_out, int64_t steps, int64_t batch, int64_t input,
                      int64_t hidden, tc_stream_t stream);

/* The same chain with caller-provided scratch memory: the input projections x_t W^T of all steps are
 * computed first as one large GEMM into `workspace` (fp32 [steps, batch, 4*hidden], 16-byte aligned,
 * tc_lstm_chain_workspace_bytes() bytes) and each step only runs the recurrent product h U^T. Same
 * results as tc_lstm_chain_f16 up to fp32 summation order. No counterpart in the reference
 * (Makefile:3 only names test_lstm_cell). */
int64_t tc_lstm_chain_workspace_bytes(int64_t steps, int64_t batch, int64_t hidden);
int tc_lstm_chain_ws_f16(const void* W, const void* U, const float* bias, const void* x, const void* h0,
                         const float* c0, void* h_all, float* c_out, int64_t steps, int64_t batch, int64_t input,
                         int64_t hidden, void* workspace, int64_t workspace_bytes, tc_stream_t stream);

/* The chain of tc_lstm_chain_ws_f16 for callers that cannot allocate device memory or hand over scratch:
 * code running under a stream capture, loops whose memory was budgeted at start-up, plug-ins that only
 * receive input and output buffers. It calls no cudaMalloc / cudaFree and no allocating library routine.
 * Its scratch (fp32 [steps, batch, 4*hidden]) is a 64 MiB array that is part of the library image, so
 * steps * batch * 4 * hidden * 4 must not exceed 67,108,864 bytes (TC_ERR_UNSUPPORTED otherwise), and
 * every GPU that loads the library holds those 64 MiB until the library is unloaded. All calls on one
 * device share that array: calls whose kernels overlap on the GPU (different streams, or the same
 * stream from two threads) race on it; run them one after the other. The first call on a device looks
 * up the array's device address, and the first call with a given shape class (batch above or below 128
 * rows per tile, hidden size, the tile plan of the hoisted GEMM) sets the shared-memory limits of the
 * kernels it picks; make a first call with the shapes you will use before any stream capture begins. A call with
 * steps == 0 launches nothing: it synchronises the device and returns TC_ERR_DEVICE if a kernel of an
 * earlier call of this entry point recorded a timeout (tc_device_status() does not cover this path).
 * Arguments otherwise as tc_lstm_chain_f16. It has no counterpart in the reference. */
int tc_lstm_chain_static_f16(const void* W, const void* U, const float* bias, const void* x, const void* h0,
                             const float* c0, void* h_all, float* c_out, int64_t steps, int64_t batch, int64_t input,
                             int64_t hidden, tc_stream_t stream);

/* ScatterND assignment: for each of the n index tuples t (k integers each, int64 when idx_is_int64
 * else int32), data[idx[t,0], ..., idx[t,k-1], :] = updates[t, :], where data has `rank` dimensions
 * `dims` (row-major, elements of elem_bytes bytes) and the slice is the product of dims[k..rank).
 * Tuples must be unique for a deterministic result; out-of-range tuples are skipped and reported
 * through tc_device_status(). Tables larger than 2^32 elements are fine (64-bit offsets).
 * Replaces `scatter_nd_kernel` / `scatter_nd<T>` / `custom_scatter_op`
 * (src/kernels/scatter_nd.cu:25-50, 52-112, 114-122) with the assignment semantics of the reference's
 * own test oracle (tests/python/test_scatter_nd.py:46). */
int tc_scatter_nd(void* data, const void* updates, const void* indices, int idx_is_int64, const int64_t* dims,
                  int rank, int64_t n, int k, int elem_bytes, tc_stream_t stream);

/* ScatterND accumulation: data[idx[t,0], ..., idx[t,k-1], :] += updates[t, :]; repeated tuples add up (in
 * an unspecified order, so floating-point sums of repeated tuples may differ in the last bits from run
 * to run; int32 sums are exact). elem_type: 0 = fp32, 1 = fp16, 2 = int32, 3 = fp64. Other arguments and
 * the treatment of out-of-range tuples as tc_scatter_nd. This is what the reference's kernel does
 * element by element with atomicAdd (src/kernels/scatter_nd.cu:25-50, the additions at :44-47), whereas
 * its test oracle (tests/python/test_scatter_nd.py:46) assigns. */
int tc_scatter_nd_add(void* data, const void* updates, const void* indices, int idx_is_int64, const int64_t* dims,
                      int rank, int64_t n, int k, int elem_type, tc_stream_t stream);

/* Peer windows, for assembling sharded outputs inside one box with one process per GPU: a rank exports a device
 * buffer, the other ranks open it and copy their finished blocks straight into it over NVLink on the copy engines
 * (no SM is taken from the kernels that run beside the copy). tc_peer_export writes an opaque handle of
 * TC_PEER_HANDLE_BYTES bytes that names the whole device allocation dev_ptr lies in; the handle travels to the other
 * processes by any host channel. tc_peer_open, called with the opener's own compute device current, returns the base
 * address of that allocation as seen from the opener (add the exported pointer's offset inside its allocation);
 * an allocation can be opened once per process. tc_peer_copy queues a device-to-device copy on `stream`; ordering
 * against the owner's own kernels is the caller's business (a collective or an event shared by the ranks).
 * tc_peer_close unmaps a window; every rank closes its windows on a buffer before the owner frees it. The reference is
 * single-GPU and single-process; these have no counterpart there. */
#define TC_PEER_HANDLE_BYTES 64
int tc_peer_export(const void* dev_ptr, void* handle_out, int64_t handle_bytes);
int tc_peer_open(const void* handle, int64_t handle_bytes, void** base_out);
int tc_peer_close(void* base);
int tc_peer_copy(void* dst, const void* src, int64_t bytes, tc_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TILEDCUDA_B200_H_ */
