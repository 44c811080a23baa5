// Device-side primitives for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (MMA, TMEM
// allocation, TMEM load/store) and the shared-memory / instruction descriptors that tcgen05.mma takes.
//
// Every wait in this file is bounded: a wait that runs out sets a CTA-wide abort word and returns
// false; callers leave their loops, the CTA frees its TMEM and the host finds the code in the device
// status word. Nothing here traps or asserts.
#pragma once

#include <cuda.h>  // CUtensorMap (type only; the driver is reached through the runtime)
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tcb {

// ---- status codes written by kernels into the device status word -------------------------------
enum DeviceStatus : uint32_t {
    kDevOk = 0,
    kDevTimeoutProducer = 1,   // TMA producer waited too long for a free stage
    kDevTimeoutMma = 2,        // MMA issuer waited too long for operands / a free accumulator
    kDevTimeoutEpilogue = 3,   // epilogue waited too long for an accumulator
    kDevTimeoutSoftmax = 4,    // softmax warps waited too long
    kDevIndexOutOfRange = 16,  // scatter_nd met an index outside the table
};

constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s: far above any legitimate wait here

// ---- small helpers -------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }

// ---- programmatic dependent launch ---------------------------------------------------------------
// wait: blocks until the grids this launch depends on have completed and their writes are visible (a no-op
// when the launch carries no programmatic dependency). launch_dependents: lets the next launch in the stream
// begin its own prologue while this grid is still running.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- mbarrier ------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

// Makes barrier initialisation visible to the async proxy (TMA, tcgen05.commit).
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Orders generic-proxy writes to shared memory before later async-proxy reads (tcgen05.mma, TMA store).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

// Non-blocking test of a phase (mbarrier.test_wait never suspends the thread; try_wait may, for a
// hardware-chosen time, when the phase is not complete yet).
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded waits. The common case, a phase that is already complete or completes within a few polls, must
// cost no more than the poll itself (about a dozen cycles): the fast path is a single try_wait and a
// uniform branch, and everything that needs a loop, the clock or the abort word lives in a separate
// non-inlined function, so that the caller carries none of its control flow.
//
// mbar_wait: one thread. Returns false when another role has aborted or when the limit ran out (then it
// records `code` in the CTA's abort word).
static __device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_word,
                                            uint32_t code) {
    uint32_t it = 0;
    uint64_t t0 = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++it & 0xfffu) == 0) {
            if (*abort_word != 0) return false;
            const uint64_t now = global_timer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > kWaitLimitNs) {
                *abort_word = code;
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_word,
                                          uint32_t code) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_word, code);
}

// mbar_wait_warp: a whole converged warp; every lane polls (so every lane acquires the phase) and the
// warp leaves together, which keeps a timeout from leaving part of a warp behind before a
// warp-collective instruction (tcgen05.ld / st, votes).
static __device__ __noinline__ bool mbar_wait_warp_slow(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_word,
                                                 uint32_t code) {
    uint32_t it = 0;
    uint64_t t0 = 0;
    while (!__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) {
        if ((++it & 0xfffu) == 0) {
            uint32_t give_up = 0;
            if (*abort_word != 0) {
                give_up = 1;
            } else {
                const uint64_t now = global_timer_ns();
                if (t0 == 0) {
                    t0 = now;
                } else if (now - t0 > kWaitLimitNs) {
                    *abort_word = code;
                    give_up = 1;
                }
            }
            if (__any_sync(0xffffffffu, give_up)) return false;
        }
    }
    return true;
}

__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_word,
                                               uint32_t code) {
    if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
    return mbar_wait_warp_slow(bar, parity, abort_word, code);
}

// ---- TMA -----------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// 2-D tile load, no multicast: lands in this CTA's shared memory and completes on this CTA's barrier.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y,
                                            int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], "
        "[%2];" ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y,
                                            int z, int w) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
        "[%2];" ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}

// 2-D tile store shared -> global (bulk async group).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(m)),
                 "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, const void* smem_src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(m)),
                 "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, const void* smem_src, int x, int y, int z, int w) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(m)),
                 "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z), "r"(w)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---- CTA pairs (cluster of two) --------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// Address of the same shared-memory location in CTA `rank` of this cluster (shared::cluster window).
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}

// Hardware barrier over all threads of the cluster. Bounded by construction: every thread of both CTAs
// reaches it because every wait before it is bounded.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Arrive on a barrier that lives in another CTA of the cluster (address from map_to_cta).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// 2-D tile load issued by either CTA of a pair for a pair-wide MMA: the data lands in the issuing CTA's
// shared memory, the byte count completes on `bar_cluster_addr`, which may be the leader CTA's barrier.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x,
                                                 int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}

// Pair-wide TMEM allocation: one warp of EACH CTA of the pair executes it, with the same slot offset.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// Pair-wide MMA, issued by one thread of the leader CTA (even rank): D[256 x N] (+)= A[256 x 16] B[16 x N].
// Each CTA supplies its 128 rows of A and its N/2 rows of B at the same shared-memory offsets and holds
// its 128 rows of D in its own TMEM at the same address.
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 bool accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate))
        : "memory");
}

// Arrives once on the barrier at `bar_cluster_addr` (own or peer CTA) when every pair-wide MMA issued so far
// by this thread has completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
                 : "memory");
}

// The same arrival on the barrier at this shared-memory offset in BOTH CTAs of the pair with one instruction
// (a commit multicast; no data is loaded).
__device__ __forceinline__ void umma_commit_pair_both(uint32_t bar_cta_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                     bar_cta_addr),
                 "h"(static_cast<uint16_t>(3))
                 : "memory");
}

// ---- tcgen05: TMEM allocation ---------------------------------------------------------------------
// Executed by one whole warp. `cols` is a power of two in [32, 512]. The base address lands in *slot.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- tcgen05: descriptors ---------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle. The tile must start on a 1024-byte boundary
// (plus a multiple of 32 bytes when stepping along K inside a swizzle row).
//   K-major operand: rows of 64 fp16 (128 B); 8 rows form a 1024-B swizzle atom; `sbo` is the
//     byte distance between consecutive 8-row groups (1024 for a dense tile); `lbo` is ignored.
//   MN-major operand: 64 fp16 along M/N are contiguous (128 B); 8 consecutive K rows form a 1024-B
//     atom; `sbo` = distance between 8-row K groups, `lbo` = distance between 64-element M/N groups.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);           // bits [0,14): start address / 16
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;      // bits [16,30): leading byte offset / 16
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;      // bits [32,46): stride byte offset / 16
    d |= static_cast<uint64_t>(1) << 46;                               // bits [46,48): descriptor version 1
    d |= static_cast<uint64_t>(2) << 61;                               // bits [61,64): 128-byte swizzle
    return d;
}

// The same descriptor split into its two 32-bit words. Only the low word depends on the address, so an
// issuing thread can build the high word once and form each descriptor with one add: stepping the start
// address by `bytes` adds bytes / 16 to the low word (no carry out of the 14-bit field below 256 KiB).
__device__ __forceinline__ uint32_t smem_desc_hi_sw128(uint32_t sbo_bytes) {
    return ((sbo_bytes >> 4) & 0x3fffu) | (1u << 14) | (2u << 29);
}
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t smem_addr, uint32_t lbo_bytes) {
    return ((smem_addr & 0x3ffffu) >> 4) | (((lbo_bytes >> 4) & 0x3fffu) << 16);
}
__device__ __forceinline__ uint64_t smem_desc_join(uint32_t lo, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}

// Instruction descriptor for kind::f16: fp16 A and B, fp32 accumulate.
//   bits [4,6) D format (1 = f32), [7,10) A format (0 = f16), [10,13) B format (0 = f16),
//   bit 15 A major (0 = K), bit 16 B major (0 = K, 1 = MN), [17,23) N/8, [24,29) M/16.
__host__ __device__ constexpr uint32_t make_idesc_f16_f32(int m, int n, bool a_mn_major, bool b_mn_major) {
    return (1u << 4) | (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// OR-ed into an instruction descriptor to declare A and B as bf16 instead of fp16 (format field value 1).
constexpr uint32_t kIdescBf16Inputs = (1u << 7) | (1u << 10);

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            bool accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate))
        : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]: A is read from TMEM (row r in lane r; K runs along the columns, two
// fp16 per 32-bit column, even K index in the low half), so K = 16 spans 8 columns. Issued by one thread.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            bool accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate))
        : "memory");
}

// True in exactly one lane of a converged warp (the same lane on every call).
__device__ __forceinline__ bool elect_one_sync() {
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(pred));
    return pred != 0;
}

// Arrives once on `bar` when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// ---- tcgen05: TMEM <-> registers --------------------------------------------------------------------
// 32x32b shape: lane i of the warp reads TMEM lane (base lane + i); register j is column (base col + j).
// A warp may only touch the 32 TMEM lanes of its quarter: lanes 32*(warp_id % 4) .. +31.
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- misc math ----------------------------------------------------------------------------------------
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- packed fp32 pairs: one instruction does the arithmetic of two values (sm_100: add / mul / fma .f32x2) ----
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t add2_round_down(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rm.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

// 2^x of two values on the FMA pipe, for x <= ~100: floor(x) by the round-down magic-number add, a degree-3 minimax
// polynomial for 2^frac on [0, 1) (max relative error 7.5e-5, below fp16 resolution), and the integer part
// added into the exponent field. Takes load off the 16-lane special-function unit, which the exponentials of an
// attention tile otherwise saturate. xa and xb are the two halves of x2 (the caller has them unpacked anyway).
__device__ __forceinline__ void poly_exp2_pair(float xa, float xb, float& a, float& b) {
    const uint64_t magic = pack2(12582912.f, 12582912.f);   // 1.5 * 2^23: the low mantissa bits of the sum hold floor(x)
    const uint64_t xc = pack2(fmaxf(xa, -126.f), fmaxf(xb, -126.f));
    const uint64_t y = add2_round_down(xc, magic);
    const uint64_t fl = add2(y, pack2(-12582912.f, -12582912.f));
    const uint64_t f = fma2(fl, pack2(-1.f, -1.f), xc);
    uint64_t q = fma2(pack2(0.07802422344684601f, 0.07802422344684601f), f, pack2(0.22606723010540009f, 0.22606723010540009f));
    q = fma2(q, f, pack2(0.695833683013916f, 0.695833683013916f));
    q = fma2(q, f, pack2(0.9999251961708069f, 0.9999251961708069f));
    float qa, qb, ya, yb;
    unpack2(q, qa, qb);
    unpack2(y, ya, yb);
    a = __int_as_float(__float_as_int(qa) + (__float_as_int(ya) << 23));
    b = __int_as_float(__float_as_int(qb) + (__float_as_int(yb) << 23));
}

// max of three (one instruction on sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float fmin3(float a, float b, float c) {
    float d;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Byte offset of the 16-byte chunk `chunk16` (0..7) of row `row` inside a K-major 128-byte-swizzled tile
// whose rows are 128 bytes long (the layout TMA writes with 128B swizzle and tcgen05.mma reads).
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t chunk16) {
    return (row >> 3) * 1024u + (row & 7u) * 128u + ((chunk16 ^ (row & 7u)) << 4);
}

// Dynamic shared memory rounded up to a 1024-byte boundary (128B-swizzle tiles need it).
__device__ __forceinline__ uint8_t* align_smem_1024(uint8_t* raw) {
    const uint32_t a = smem_u32(raw);
    return raw + ((1024u - (a & 1023u)) & 1023u);
}

}  // namespace tcb
