// Test kernels written against the tile API headers (tiledcuda_b200/include), the way a user of the
// library writes kernels: declare tile types, iterate, load, multiply, store. Each kernel is one CTA of
// 128 threads, like the single-CTA kernels of the reference's unit tests (tests/cpp/cell/test_gemm.cu,
// test_g2s_load.cu, test_swizzled_copy.cu, test_softmax.cu, test_reduce.cu, test_broadcast.cu), whose
// shapes the Python tests replay. Results are copied back and compared on the host: nothing here asserts
// or traps on the device. A kernel that gives up on a bounded wait writes 1 to *status.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "cell/mod.hpp"
#include "types/mod.hpp"

using namespace tiledcuda::cell;
namespace tl = tiledcuda::cell::tile_layout;
using WarpLayout = tl::RowMajor<4, 1>;

__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
    return p + ((1024u - (a & 1023u)) & 1023u);
}

// ------------------------------------------------------------------------------------ copy round trip
// global -> shared (operand or plain layout) -> global; must reproduce the input exactly.
template <typename T, typename GLayout, bool kSwizzled>
__global__ void k_roundtrip(const T* in, T* out) {
    extern __shared__ uint8_t raw[];
    using Global = GlobalTile<T, GLayout>;
    using Shared = SharedTile<T, GLayout, kSwizzled>;
    Shared s(reinterpret_cast<T*>(align1024(raw)));
    Global gin(in), gout(out);
    copy::GlobalToSharedLoader<Shared, WarpLayout> load;
    copy::SharedToGlobalStorer<Shared, WarpLayout> store;
    load(gin, s);
    __copy_async();
    __syncthreads();
    store(s, gout);
}

// global -> shared -> global through a GTileIterator, chunk by chunk: the shapes of the reference's swizzled-load
// tests (tests/cpp/cell/test_swizzled_copy.cu:399-449). Each chunk goes into a shared operand tile (128-byte
// swizzle or interleaved core matrices) and back out to the same chunk of the output.
template <typename GLayout, typename ChunkShape, typename SLayout, bool kSwizzled>
__global__ void k_chunked_roundtrip(const __half* in, __half* out) {
    extern __shared__ uint8_t raw[];
    using Global = GlobalTile<__half, GLayout>;
    using GIter = GTileIterator<Global, ChunkShape>;
    using Shared = SharedTile<__half, SLayout, kSwizzled>;
    Shared s(reinterpret_cast<__half*>(align1024(raw)));
    GIter gin(in), gout(out);
    copy::GlobalToSharedLoader<Shared, WarpLayout> load;
    copy::SharedToGlobalStorer<Shared, WarpLayout> store;
    constexpr int kChunks = GIter::sc0 * GIter::sc1;
    for (int i = 0; i < kChunks; ++i) {
        auto src = gin(i);
        auto dst = gout(i);
        load(src, s);
        __copy_async();
        __syncthreads();
        store(s, dst);
        __syncthreads();
    }
}

// ------------------------------------------------------------------------------------ tile GEMM
// C[M,N] = A[M,K] B[K,N] with A row-major, B column-major, fp32 C, K walked in chunks of TK.
template <int M, int N, int K, int TK, bool kSwizzled>
__global__ void k_tile_gemm(const __half* dA, const __half* dB, float* dC, int* status) {
    extern __shared__ uint8_t raw[];
    using GlobalA = GlobalTile<__half, tl::RowMajor<M, K>>;
    using GlobalB = GlobalTile<__half, tl::ColMajor<K, N>>;
    using GlobalC = GlobalTile<float, tl::RowMajor<M, N>>;
    using IterA = GTileIterator<GlobalA, TileShape<M, TK>>;
    using IterB = GTileIterator<GlobalB, TileShape<TK, N>>;
    using SharedA = SharedTile<__half, tl::RowMajor<M, TK>, kSwizzled>;
    using SharedB = SharedTile<__half, tl::ColMajor<TK, N>, kSwizzled>;
    using Acc = TmemTile<float, tl::RowMajor<128, N>>;
    using RegC = RowFragment<float, N>;

    uint8_t* smem = align1024(raw);
    SharedA sA(reinterpret_cast<__half*>(smem));               // 64 KiB reserved: the MMA always reads 128 rows
    SharedB sB(reinterpret_cast<__half*>(smem + 64 * 1024));   // up to 256 x 128 fp16 = 64 KiB
    uint64_t* bar_mem = reinterpret_cast<uint64_t*>(smem + 128 * 1024);
    uint32_t* slot = reinterpret_cast<uint32_t*>(bar_mem + 1);

    MmaBarrier bar(bar_mem);
    if (threadIdx.x == 0) bar.init();
    if (threadIdx.x < 32) copy::TmemAllocator::alloc(slot, tmem_alloc_columns(N));
    __syncthreads();
    Acc acc(*slot);

    IterA gAs(dA);
    IterB gBs(dB);
    copy::GlobalToSharedLoader<SharedA, WarpLayout> load_a;
    copy::GlobalToSharedLoader<SharedB, WarpLayout> load_b;
    bool ok = true;
    for (int k = 0; k < IterA::sc1; ++k) {
        load_a(gAs(k), sA);
        load_b(gBs(k), sB);
        __copy_async();
        __syncthreads();
        compute::gemm(sA, sB, acc, k > 0);
        if (threadIdx.x == 0) bar.commit();
        ok = bar.wait() && ok;  // operands may be overwritten and acc read after this
    }
    if (ok) {
        RegC rC;
        copy::TmemToRegLoader<Acc, RegC>{}(acc, rC);
        GlobalC gC(dC);
        copy::RegToGlobalStorer<GlobalC, RegC, WarpLayout>{}(rC, gC);
    } else if (threadIdx.x == 0) {
        *status = 1;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x < 32) copy::TmemAllocator::free(acc.address(), tmem_alloc_columns(N));
}

// The same product with the K slab of each global chunk (TK wide) multiplied in narrower steps of RK through two
// STileIterators, the loop of the reference's GEMM example (examples/cpp/01_gemm/02_gemm_all_mem/gemm.hpp:145-150:
// `for k2: load_rA(sAs(k2)); load_rB(sBs(k2)); gemm(rA, rB, acc)`); here the chunks are MMA operands as they are.
template <int M, int N, int K, int TK, int RK, bool kSwizzled>
__global__ void k_tile_gemm_siter(const __half* dA, const __half* dB, float* dC, int* status) {
    extern __shared__ uint8_t raw[];
    using GlobalA = GlobalTile<__half, tl::RowMajor<M, K>>;
    using GlobalB = GlobalTile<__half, tl::ColMajor<K, N>>;
    using GlobalC = GlobalTile<float, tl::RowMajor<M, N>>;
    using IterA = GTileIterator<GlobalA, TileShape<M, TK>>;
    using IterB = GTileIterator<GlobalB, TileShape<TK, N>>;
    using SharedA = SharedTile<__half, tl::RowMajor<M, TK>, kSwizzled>;
    using SharedB = SharedTile<__half, tl::ColMajor<TK, N>, kSwizzled>;
    using SIterA = STileIterator<SharedA, TileShape<M, RK>>;
    using SIterB = STileIterator<SharedB, TileShape<RK, N>>;
    using Acc = TmemTile<float, tl::RowMajor<128, N>>;
    using RegC = RowFragment<float, N>;
    static_assert(TK > RK && SIterA::sc1 == TK / RK && SIterB::sc0 == TK / RK, "the shared slab is walked in TK / RK steps");

    uint8_t* smem = align1024(raw);
    SharedA sA(reinterpret_cast<__half*>(smem));
    SharedB sB(reinterpret_cast<__half*>(smem + 64 * 1024));
    uint64_t* bar_mem = reinterpret_cast<uint64_t*>(smem + 128 * 1024);
    uint32_t* slot = reinterpret_cast<uint32_t*>(bar_mem + 1);

    MmaBarrier bar(bar_mem);
    if (threadIdx.x == 0) bar.init();
    if (threadIdx.x < 32) copy::TmemAllocator::alloc(slot, tmem_alloc_columns(N));
    __syncthreads();
    Acc acc(*slot);

    IterA gAs(dA);
    IterB gBs(dB);
    SIterA sAs(sA);
    SIterB sBs(sB);
    copy::GlobalToSharedLoader<SharedA, WarpLayout> load_a;
    copy::GlobalToSharedLoader<SharedB, WarpLayout> load_b;
    bool ok = true;
    for (int k = 0; k < IterA::sc1; ++k) {
        load_a(gAs(k), sA);
        load_b(gBs(k), sB);
        __copy_async();
        __syncthreads();
        for (int k2 = 0; k2 < SIterA::sc1; ++k2) compute::gemm(sAs(k2), sBs(k2), acc, (k | k2) != 0);
        if (threadIdx.x == 0) bar.commit();
        ok = bar.wait() && ok;
    }
    if (ok) {
        RegC rC;
        copy::TmemToRegLoader<Acc, RegC>{}(acc, rC);
        GlobalC gC(dC);
        copy::RegToGlobalStorer<GlobalC, RegC, WarpLayout>{}(rC, gC);
    } else if (threadIdx.x == 0) {
        *status = 1;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x < 32) copy::TmemAllocator::free(acc.address(), tmem_alloc_columns(N));
}

// ------------------------------------------------------------------------------------ loaders and storers
// global -> shared operand tile -> SharedToRegLoader (one row per thread, converted to Out) -> global.
template <typename Out, int R, int C, bool kSwizzled>
__global__ void k_shared_to_reg(const __half* in, Out* out) {
    extern __shared__ uint8_t raw[];
    using GlobalIn = GlobalTile<__half, tl::RowMajor<R, C>>;
    using GlobalOut = GlobalTile<Out, tl::RowMajor<R, C>>;
    using Shared = SharedTile<__half, tl::RowMajor<R, C>, kSwizzled>;
    using Reg = RowFragment<Out, C>;
    Shared s(reinterpret_cast<__half*>(align1024(raw)));
    GlobalIn gin(in);
    copy::GlobalToSharedLoader<Shared, WarpLayout>{}(gin, s);
    __copy_async();
    __syncthreads();
    Reg r;
    copy::SharedToRegLoader<Reg, WarpLayout>{}(s, r);
    GlobalOut gout(out);
    copy::RegToGlobalStorer<GlobalOut, Reg, WarpLayout>{}(r, gout);
}

// global fp32 [128, C] -> row fragments -> RegToTmemStorer -> TMEM -> TmemToRegLoader -> global.
template <int C>
__global__ void k_tmem_roundtrip(const float* in, float* out) {
    __shared__ uint32_t slot;
    using Global = GlobalTile<float, tl::RowMajor<128, C>>;
    using Reg = RowFragment<float, C>;
    using Tmem = TmemTile<float, tl::RowMajor<128, C>>;
    if (threadIdx.x < 32) copy::TmemAllocator::alloc(&slot, tmem_alloc_columns(C));
    __syncthreads();
    Tmem t(slot);
    Global gin(in), gout(out);
    Reg a, b;
    copy::GlobalToRegLoader<Reg, WarpLayout>{}(gin, a);
    copy::RegToTmemStorer<Reg, Tmem>{}(a, t);
    __syncthreads();
    copy::TmemToRegLoader<Tmem, Reg>{}(t, b);
    copy::RegToGlobalStorer<Global, Reg, WarpLayout>{}(b, gout);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x < 32) copy::TmemAllocator::free(t.address(), tmem_alloc_columns(C));
}

// Tensor-map load of an R x C window at (row0, col0) of a larger fp16 matrix into a swizzled operand tile
// (TmaTileLoader, one thread), then out through SharedToGlobalStorer. The wait on the copy is bounded.
template <int R, int C>
__global__ void k_tma_load(const __grid_constant__ CUtensorMap map, int row0, int col0, __half* out, int* status) {
    extern __shared__ uint8_t raw[];
    using Shared = SharedTile<__half, tl::RowMajor<R, C>, true>;
    using Global = GlobalTile<__half, tl::RowMajor<R, C>>;
    uint8_t* smem = align1024(raw);
    Shared s(reinterpret_cast<__half*>(smem));
    CopyBarrier bar(reinterpret_cast<uint64_t*>(smem + Shared::kBytes));
    if (threadIdx.x == 0) {
        bar.init();
        bar.expect(Shared::kBytes);
        copy::TmaTileLoader<Shared>{}(&map, s, bar.get(), col0, row0);
    }
    __syncthreads();
    if (bar.wait()) {
        Global gout(out);
        copy::SharedToGlobalStorer<Shared, WarpLayout>{}(s, gout);
    } else if (threadIdx.x == 0) {
        *status = 1;
    }
}

// ------------------------------------------------------------------------------------ a wait that runs out
// One CTA allocates TMEM and waits, with a limit of `limit_ns`, on an MMA barrier that nothing ever commits. The
// wait gives up, every thread sees `false`, the CTA frees its TMEM, records status 1 and returns: the way every
// kernel of the library leaves when a wait runs out. The context stays usable; nothing traps.
__global__ void k_wait_runs_out(unsigned long long limit_ns, int* status, unsigned long long* waited_ns) {
    __shared__ uint64_t bar_mem;
    __shared__ uint32_t slot;
    MmaBarrier bar(&bar_mem);
    if (threadIdx.x == 0) bar.init();
    if (threadIdx.x < 32) copy::TmemAllocator::alloc(&slot, 32);
    __syncthreads();
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    const bool ok = bar.wait(limit_ns);
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    if (threadIdx.x == 0) {
        *status = ok ? 0 : 1;
        *waited_ns = t1 - t0;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x < 32) copy::TmemAllocator::free(slot, 32);
}

// ------------------------------------------------------------------------------------ fused two GEMMs
// E[M,P] = fp16(A[M,K] B[K,N]) D[N,P], the intermediate going TMEM -> registers -> fp16 -> shared operand tile
// (the structure of the reference's KeFusedGemm, examples/cpp/02_fused_two_gemms/fused_gemm.hpp:152-180).
template <int M, int N, int K, int P>
__global__ void k_tile_b2b(const __half* dA, const __half* dB, const __half* dD, float* dE, int* status) {
    extern __shared__ uint8_t raw[];
    using GlobalA = GlobalTile<__half, tl::RowMajor<M, K>>;
    using GlobalB = GlobalTile<__half, tl::ColMajor<K, N>>;
    using GlobalD = GlobalTile<__half, tl::ColMajor<N, P>>;
    using GlobalE = GlobalTile<float, tl::RowMajor<M, P>>;
    using SharedA = SharedTile<__half, tl::RowMajor<M, K>, true>;
    using SharedB = SharedTile<__half, tl::ColMajor<K, N>, true>;
    using SharedD = SharedTile<__half, tl::ColMajor<N, P>, true>;
    using SharedS = SharedTile<__half, tl::RowMajor<128, N>, true>;  // the intermediate as operand A of the second product
    using AccS = TmemTile<float, tl::RowMajor<128, N>>;
    using AccE = TmemTile<float, tl::RowMajor<128, P>>;

    uint8_t* smem = align1024(raw);
    SharedA sA(reinterpret_cast<__half*>(smem));
    SharedB sB(reinterpret_cast<__half*>(smem + 32 * 1024));
    SharedD sD(reinterpret_cast<__half*>(smem + 64 * 1024));
    SharedS sS(reinterpret_cast<__half*>(smem + 96 * 1024));
    uint64_t* bar_mem = reinterpret_cast<uint64_t*>(smem + 128 * 1024);
    uint32_t* slot = reinterpret_cast<uint32_t*>(bar_mem + 1);

    MmaBarrier bar(bar_mem);
    if (threadIdx.x == 0) bar.init();
    if (threadIdx.x < 32) copy::TmemAllocator::alloc(slot, tmem_alloc_columns(N + P));
    __syncthreads();
    AccS accS(*slot);
    AccE accE(*slot + N);

    GlobalA gA(dA);
    GlobalB gB(dB);
    GlobalD gD(dD);
    copy::GlobalToSharedLoader<SharedA, WarpLayout>{}(gA, sA);
    copy::GlobalToSharedLoader<SharedB, WarpLayout>{}(gB, sB);
    copy::GlobalToSharedLoader<SharedD, WarpLayout>{}(gD, sD);
    __copy_async();
    __syncthreads();

    compute::gemm(sA, sB, accS, false);
    if (threadIdx.x == 0) bar.commit();
    bool ok = bar.wait();

    RowFragment<float, N> rS;
    copy::TmemToRegLoader<AccS, RowFragment<float, N>>{}(accS, rS);
    copy::RegToSharedStorer<RowFragment<float, N>, WarpLayout>{}(rS, sS);  // rounds to fp16, writes the swizzled operand layout
    fence_async_proxy();
    __syncthreads();

    compute::gemm(sS, sD, accE, false);
    if (threadIdx.x == 0) bar.commit();
    ok = bar.wait() && ok;
    if (ok) {
        RowFragment<float, P> rE;
        copy::TmemToRegLoader<AccE, RowFragment<float, P>>{}(accE, rE);
        GlobalE gE(dE);
        copy::RegToGlobalStorer<GlobalE, RowFragment<float, P>, WarpLayout>{}(rE, gE);
    } else if (threadIdx.x == 0) {
        *status = 1;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x < 32) copy::TmemAllocator::free(accS.address(), tmem_alloc_columns(N + P));
}

// ------------------------------------------------------------------------------------ tile flash attention
// O[M,P] = softmax(Q K^T) V for one tile of M <= 128 query rows, KV walked in blocks of BN with two GTileIterators,
// written with the tile vocabulary only and following the reference's recurrence statement for statement
// (tests/python/test_flash_attn.py:27-75; examples/cpp/03_flash_attention/flash_attn.hpp): per block
//   cur_max = rowmax(S); E = exp(S - cur_max); cur_sum = rowsum(E); new_max = max(cur_max, prev_max);
//   renorm_prev = exp(prev_max - new_max); renorm_cur = exp(cur_max - new_max);
//   new_sum = renorm_prev prev_sum + renorm_cur cur_sum; O = (O prev_sum renorm_prev + renorm_cur (E V)) / new_sum.
// Q is row-major [M,K], K the column-major [K,N] operand (stored [N,K]), V the column-major [N,P] operand (stored
// [P,N]), as the reference's kernel takes them. fp32 statistics; E is rounded to fp16 for the second product.
template <int M, int N, int K, int P, int BN>
__global__ void k_tile_flash_attn(const __half* dQ, const __half* dK, const __half* dV, float* dO, int* status) {
    extern __shared__ uint8_t raw[];
    using GlobalQ = GlobalTile<__half, tl::RowMajor<M, K>>;
    using GlobalK = GlobalTile<__half, tl::ColMajor<K, N>>;
    using GlobalV = GlobalTile<__half, tl::ColMajor<N, P>>;
    using GlobalO = GlobalTile<float, tl::RowMajor<M, P>>;
    using IterK = GTileIterator<GlobalK, TileShape<K, BN>>;
    using IterV = GTileIterator<GlobalV, TileShape<BN, P>>;
    using SharedQ = SharedTile<__half, tl::RowMajor<M, K>, true>;
    using SharedK = SharedTile<__half, tl::ColMajor<K, BN>, true>;
    using SharedV = SharedTile<__half, tl::ColMajor<BN, P>, true>;
    using SharedE = SharedTile<__half, tl::RowMajor<128, BN>, true>;
    using AccS = TmemTile<float, tl::RowMajor<128, BN>>;
    using AccO = TmemTile<float, tl::RowMajor<128, P>>;
    using RegS = RowFragment<float, BN>;
    using RegO = RowFragment<float, P>;
    using Val = RowScalar<float>;

    uint8_t* smem = align1024(raw);
    SharedQ sQ(reinterpret_cast<__half*>(smem));
    SharedK sK(reinterpret_cast<__half*>(smem + 32 * 1024));
    SharedV sV(reinterpret_cast<__half*>(smem + 64 * 1024));
    SharedE sE(reinterpret_cast<__half*>(smem + 96 * 1024));
    uint64_t* bar_mem = reinterpret_cast<uint64_t*>(smem + 128 * 1024);
    uint32_t* slot = reinterpret_cast<uint32_t*>(bar_mem + 1);

    MmaBarrier bar(bar_mem);
    if (threadIdx.x == 0) bar.init();
    if (threadIdx.x < 32) copy::TmemAllocator::alloc(slot, tmem_alloc_columns(BN + P));
    __syncthreads();
    AccS accS(*slot);
    AccO accEV(*slot + BN);

    GlobalQ gQ(dQ);
    IterK gKs(dK);
    IterV gVs(dV);
    copy::GlobalToSharedLoader<SharedQ, WarpLayout>{}(gQ, sQ);

    RegS rS, rE;
    RegO rO, rEV;
    Val prev_max, prev_sum, cur_max, cur_sum, new_max, new_sum, renorm_prev, renorm_cur, tmp;
    rO.clear();
    prev_max.clear();
    prev_sum.clear();
    bool ok = true;

    for (int j = 0; j < N / BN; ++j) {
        auto gK = gKs(j);
        auto gV = gVs(j);
        copy::GlobalToSharedLoader<SharedK, WarpLayout>{}(gK, sK);
        copy::GlobalToSharedLoader<SharedV, WarpLayout>{}(gV, sV);
        __copy_async();
        __syncthreads();

        compute::gemm(sQ, sK, accS, false);
        if (threadIdx.x == 0) bar.commit();
        ok = bar.wait() && ok;
        copy::TmemToRegLoader<AccS, RegS>{}(accS, rS);

        compute::MaxReduce<RegS>{}(rS, cur_max);
        copy::copy(rS, rE);
        compute::BroadcastSub<Val, RegS>{}(cur_max, rE);
        compute::RegTileExp<RegS>{}(rE, rE);
        compute::SumReduce<RegS>{}(rE, cur_sum);

        compute::RegTileMax<Val>{}(cur_max, prev_max, new_max);
        compute::RegTileSub<Val>{}(prev_max, new_max, renorm_prev);
        compute::RegTileExp<Val>{}(renorm_prev, renorm_prev);
        compute::RegTileSub<Val>{}(cur_max, new_max, renorm_cur);
        compute::RegTileExp<Val>{}(renorm_cur, renorm_cur);
        compute::RegTileMul<Val>{}(renorm_prev, prev_sum, tmp);          // renorm_prev * prev_sum
        compute::RegTileMul<Val>{}(renorm_cur, cur_sum, new_sum);
        compute::RegTileAdd<Val>{}(new_sum, tmp, new_sum);

        copy::RegToSharedStorer<RegS, WarpLayout>{}(rE, sE);   // rounds to fp16, writes the operand layout
        fence_async_proxy();
        __syncthreads();
        compute::gemm(sE, sV, accEV, false);
        if (threadIdx.x == 0) bar.commit();
        ok = bar.wait() && ok;
        copy::TmemToRegLoader<AccO, RegO>{}(accEV, rEV);

        compute::BroadcastMul<Val, RegO>{}(tmp, rO);             // O * prev_sum * renorm_prev
        compute::BroadcastMul<Val, RegO>{}(renorm_cur, rEV);
        compute::RegTileAdd<RegO>{}(rO, rEV, rO);
        compute::BroadcastDiv<Val, RegO>{}(new_sum, rO);
        copy::copy(new_sum, prev_sum);
        copy::copy(new_max, prev_max);
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();   // sK, sV and sE are rewritten by the next block
    }
    if (ok) {
        GlobalO gO(dO);
        copy::RegToGlobalStorer<GlobalO, RegO, WarpLayout>{}(rO, gO);
    } else if (threadIdx.x == 0) {
        *status = 1;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x < 32) copy::TmemAllocator::free(accS.address(), tmem_alloc_columns(BN + P));
}

// ------------------------------------------------------------------------------------ row operations
// in [128, C] fp32 -> softmax rows, row max, row sum, (x - max) broadcast, exp, per-warp column sums.
template <int C>
__global__ void k_row_ops(const float* in, float* softmax_out, float* row_max, float* row_sum, float* centered, float* col_sum) {
    using Global = GlobalTile<float, tl::RowMajor<128, C>>;
    using Reg = RowFragment<float, C>;
    using Val = RowScalar<float>;
    Global gin(in);
    Reg x, y;
    copy::GlobalToRegLoader<Reg, WarpLayout>{}(gin, x);
    Val mx, sm;
    compute::MaxReduce<Reg>{}(x, mx);
    compute::SumReduce<Reg>{}(x, sm);
    row_max[threadIdx.x] = mx(0, 0);
    row_sum[threadIdx.x] = sm(0, 0);
    compute::Softmax<Reg>{}(x, y);
    Global gsoft(softmax_out);
    copy::RegToGlobalStorer<Global, Reg, WarpLayout>{}(y, gsoft);
    copy::copy(x, y);
    compute::BroadcastSub<Val, Reg>{}(mx, y);
    Global gcent(centered);
    copy::RegToGlobalStorer<Global, Reg, WarpLayout>{}(y, gcent);
    Reg cs;
    compute::SumReduce<Reg, tl::Layout::kColMajor>{}(x, cs);   // sums over the 32 rows of this warp
    if ((threadIdx.x & 31) == 0)
        for (int j = 0; j < C; ++j) col_sum[(threadIdx.x >> 5) * C + j] = cs(0, j);
}

// ------------------------------------------------------------------------------------ C entry points
template <typename Kernel>
static int set_smem(Kernel k, int bytes) {
    return cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess ? 0 : -1;
}

#define GEMM_CASE(id, M, N, K, TK, SWZ)                                                   \
    case id: {                                                                            \
        auto kern = k_tile_gemm<M, N, K, TK, SWZ>;                                        \
        if (set_smem(kern, 130 * 1024 + 1024)) return -3;                                 \
        kern<<<1, 128, 130 * 1024 + 1024>>>(A, B, C, status);                             \
        *m = M; *n = N; *k = K;                                                           \
        break;                                                                            \
    }

// Shapes of the reference's test_gemm.cu:306-351 (M, N, K, chunk K), each with and without swizzle where the
// chunk is a whole number of 64-element swizzle rows.
extern "C" int tcx_gemm_case_count() { return 43; }
extern "C" int tcx_tile_gemm(int id, const __half* A, const __half* B, float* C, int* status, int* m, int* n, int* k) {
    switch (id) {
        GEMM_CASE(0, 16, 16, 16, 16, false)
        GEMM_CASE(1, 16, 16, 64, 64, true)
        GEMM_CASE(2, 16, 32, 32, 32, false)
        GEMM_CASE(3, 32, 32, 64, 64, true)
        GEMM_CASE(4, 32, 64, 128, 64, true)
        GEMM_CASE(5, 32, 64, 128, 64, false)
        GEMM_CASE(6, 64, 64, 64, 64, true)
        GEMM_CASE(7, 64, 64, 64, 32, false)
        GEMM_CASE(8, 64, 128, 128, 128, true)
        GEMM_CASE(9, 64, 32, 128, 128, false)
        GEMM_CASE(10, 96, 48, 128, 64, true)
        GEMM_CASE(11, 96, 48, 256, 64, false)
        GEMM_CASE(12, 128, 128, 64, 64, true)
        GEMM_CASE(13, 128, 128, 64, 64, false)
        GEMM_CASE(14, 128, 128, 128, 32, false)
        GEMM_CASE(15, 128, 128, 256, 128, true)
        GEMM_CASE(16, 128, 64, 512, 64, true)
        GEMM_CASE(17, 128, 256, 128, 64, true)
        GEMM_CASE(18, 128, 256, 64, 16, false)
        GEMM_CASE(19, 64, 256, 256, 128, true)
        GEMM_CASE(20, 128, 80, 192, 64, true)
        GEMM_CASE(21, 48, 112, 96, 16, false)
        // the remaining (M, N, K, K chunk) shapes of tests/cpp/cell/test_gemm.cu:312-350
        GEMM_CASE(22, 32, 16, 16, 16, true)
        GEMM_CASE(23, 16, 32, 16, 16, false)
        GEMM_CASE(24, 16, 16, 32, 16, true)
        GEMM_CASE(25, 16, 16, 32, 32, false)
        GEMM_CASE(26, 16, 32, 32, 16, true)
        GEMM_CASE(27, 32, 32, 32, 16, false)
        GEMM_CASE(28, 32, 32, 32, 32, true)
        GEMM_CASE(29, 32, 64, 32, 16, false)
        GEMM_CASE(30, 32, 64, 32, 32, true)
        GEMM_CASE(31, 32, 64, 64, 16, false)
        GEMM_CASE(32, 32, 64, 64, 32, true)
        GEMM_CASE(33, 32, 16, 32, 16, false)
        GEMM_CASE(34, 64, 32, 32, 16, true)
        GEMM_CASE(35, 64, 32, 128, 32, false)
        GEMM_CASE(36, 32, 32, 64, 32, true)
        GEMM_CASE(37, 64, 32, 64, 32, false)
        GEMM_CASE(38, 32, 32, 128, 64, true)
        GEMM_CASE(39, 64, 64, 128, 32, false)
        GEMM_CASE(40, 64, 64, 128, 128, true)
        GEMM_CASE(41, 128, 128, 64, 32, false)
        GEMM_CASE(42, 64, 128, 128, 64, true)
        default: return -1;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

#define SGEMM_CASE(id, M, N, K, TK, RK, SWZ)                                              \
    case id: {                                                                            \
        auto kern = k_tile_gemm_siter<M, N, K, TK, RK, SWZ>;                              \
        if (set_smem(kern, 130 * 1024 + 1024)) return -3;                                 \
        kern<<<1, 128, 130 * 1024 + 1024>>>(A, B, C, status);                             \
        *m = M; *n = N; *k = K;                                                           \
        break;                                                                            \
    }

// GEMMs whose shared K slab (TK) is walked in narrower steps (RK) with STileIterators: (M, N, K, TK, RK, swizzled).
// The cases cover steps inside one 128-byte swizzle row (RK = 16, 32), steps of whole swizzle rows (RK = 64), the
// interleaved layout, and M < 128.
extern "C" int tcx_siter_gemm_case_count() { return 6; }
extern "C" int tcx_tile_gemm_siter(int id, const __half* A, const __half* B, float* C, int* status, int* m, int* n, int* k) {
    switch (id) {
        SGEMM_CASE(0, 64, 256, 256, 64, 16, true)
        SGEMM_CASE(1, 128, 128, 256, 128, 64, true)
        SGEMM_CASE(2, 128, 64, 128, 64, 32, true)
        SGEMM_CASE(3, 64, 64, 128, 64, 16, false)
        SGEMM_CASE(4, 128, 128, 128, 128, 32, false)
        SGEMM_CASE(5, 32, 48, 256, 128, 16, true)
        default: return -1;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

#define S2R_CASE(id, OUT, R, C, SWZ)                                                      \
    case id: {                                                                            \
        auto kern = k_shared_to_reg<OUT, R, C, SWZ>;                                      \
        if (set_smem(kern, 70 * 1024)) return -3;                                         \
        kern<<<1, 128, 70 * 1024>>>(in, static_cast<OUT*>(out));                          \
        *rows = R; *cols = C; *out_elem = sizeof(OUT);                                    \
        break;                                                                            \
    }

extern "C" int tcx_shared_to_reg_case_count() { return 6; }
extern "C" int tcx_shared_to_reg(int id, const __half* in, void* out, int* rows, int* cols, int* out_elem) {
    switch (id) {
        S2R_CASE(0, __half, 128, 64, true)
        S2R_CASE(1, float, 128, 64, true)
        S2R_CASE(2, __half, 64, 128, false)
        S2R_CASE(3, float, 96, 32, false)
        S2R_CASE(4, float, 128, 128, true)
        S2R_CASE(5, __half, 16, 16, false)
        default: return -1;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int tcx_tmem_roundtrip(int cols, const float* in, float* out) {
    if (cols == 16)
        k_tmem_roundtrip<16><<<1, 128>>>(in, out);
    else if (cols == 64)
        k_tmem_roundtrip<64><<<1, 128>>>(in, out);
    else if (cols == 128)
        k_tmem_roundtrip<128><<<1, 128>>>(in, out);
    else
        return -1;
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Tensor map of a [rows, cols] fp16 row-major matrix with a box of 64 columns x box_rows rows and 128-byte swizzle,
// encoded through the runtime's driver entry point (no link-time dependency on the driver library).
static int encode_map(CUtensorMap* map, const void* base, int rows, int cols, int box_rows) {
    typedef CUresult (*Fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                           const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                           CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || fn == nullptr) return -4;
    const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(cols) * 2};
    const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estride[2] = {1, 1};
    const CUresult r = reinterpret_cast<Fn>(fn)(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), gdim, gstride, box,
                                                estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -5;
}

#define TMA_CASE(id, R, C)                                                                \
    case id: {                                                                            \
        if (int rc = encode_map(&map, in, rows, cols, R)) return rc;                      \
        auto kern = k_tma_load<R, C>;                                                     \
        if (set_smem(kern, 70 * 1024)) return -3;                                         \
        kern<<<1, 128, 70 * 1024>>>(map, row0, col0, out, status);                        \
        *tile_rows = R; *tile_cols = C;                                                   \
        break;                                                                            \
    }

// Loads the tile at (row0, col0) of the [rows, cols] matrix `in`; col0 must be a multiple of 8 (TMA's 16-byte rule).
extern "C" int tcx_tma_load(int id, const __half* in, int rows, int cols, int row0, int col0, __half* out, int* status,
                            int* tile_rows, int* tile_cols) {
    if (col0 % 8 != 0 || row0 < 0 || col0 < 0) return -6;
    CUtensorMap map;
    switch (id) {
        TMA_CASE(0, 64, 64)
        TMA_CASE(1, 128, 128)
        TMA_CASE(2, 32, 256)
        default: return -1;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int tcx_wait_runs_out(unsigned long long limit_ns, int* status, unsigned long long* waited_ns) {
    k_wait_runs_out<<<1, 128>>>(limit_ns, status, waited_ns);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

#define RT_CASE(id, T, LAYOUT, R, C, SWZ)                                                 \
    case id: {                                                                            \
        auto kern = k_roundtrip<T, LAYOUT<R, C>, SWZ>;                                    \
        if (set_smem(kern, 140 * 1024)) return -3;                                        \
        kern<<<1, 128, 140 * 1024>>>(static_cast<const T*>(in), static_cast<T*>(out));    \
        *rows = R; *cols = C; *elem = sizeof(T); *col_major = std::is_same_v<LAYOUT<R, C>, tl::ColMajor<R, C>>; \
        break;                                                                            \
    }

extern "C" int tcx_roundtrip_case_count() { return 42; }
extern "C" int tcx_roundtrip(int id, const void* in, void* out, int* rows, int* cols, int* elem, int* col_major) {
    switch (id) {
        RT_CASE(0, __half, tl::RowMajor, 16, 16, false)
        RT_CASE(1, __half, tl::RowMajor, 16, 64, true)
        RT_CASE(2, __half, tl::RowMajor, 64, 32, false)
        RT_CASE(3, __half, tl::RowMajor, 64, 128, true)
        RT_CASE(4, __half, tl::RowMajor, 128, 256, true)
        RT_CASE(5, __half, tl::RowMajor, 128, 256, false)
        RT_CASE(6, __half, tl::ColMajor, 64, 16, false)
        RT_CASE(7, __half, tl::ColMajor, 128, 64, true)
        RT_CASE(8, __half, tl::ColMajor, 64, 256, true)
        RT_CASE(9, float, tl::RowMajor, 16, 16, false)
        RT_CASE(10, float, tl::RowMajor, 64, 128, false)
        RT_CASE(11, float, tl::ColMajor, 128, 32, false)
        // the shapes of the reference's global-to-shared load tests (tests/cpp/cell/test_g2s_load.cu:118-143)
        RT_CASE(12, __half, tl::RowMajor, 16, 32, false)
        RT_CASE(13, __half, tl::RowMajor, 16, 32, true)
        RT_CASE(14, __half, tl::RowMajor, 32, 128, false)
        RT_CASE(15, __half, tl::RowMajor, 32, 128, true)
        RT_CASE(16, __half, tl::RowMajor, 192, 32, false)
        RT_CASE(17, __half, tl::RowMajor, 192, 32, true)
        RT_CASE(18, __half, tl::RowMajor, 64, 128, false)
        RT_CASE(19, __half, tl::RowMajor, 64, 128, true)
        RT_CASE(20, __half, tl::RowMajor, 96, 128, false)
        RT_CASE(21, __half, tl::RowMajor, 96, 128, true)
        RT_CASE(22, float, tl::RowMajor, 16, 16, false)
        RT_CASE(23, float, tl::RowMajor, 32, 128, false)
        RT_CASE(24, float, tl::RowMajor, 192, 32, false)
        RT_CASE(25, float, tl::RowMajor, 64, 128, false)
        RT_CASE(26, float, tl::RowMajor, 96, 128, false)
        RT_CASE(27, __half, tl::ColMajor, 16, 16, false)
        RT_CASE(28, __half, tl::ColMajor, 16, 16, true)
        RT_CASE(29, __half, tl::ColMajor, 32, 128, false)
        RT_CASE(30, __half, tl::ColMajor, 32, 128, true)
        RT_CASE(31, __half, tl::ColMajor, 192, 32, false)
        RT_CASE(32, __half, tl::ColMajor, 192, 32, true)
        RT_CASE(33, __half, tl::ColMajor, 64, 128, false)
        RT_CASE(34, __half, tl::ColMajor, 64, 128, true)
        RT_CASE(35, __half, tl::ColMajor, 96, 128, false)
        RT_CASE(36, __half, tl::ColMajor, 96, 128, true)
        RT_CASE(37, float, tl::ColMajor, 16, 16, false)
        RT_CASE(38, float, tl::ColMajor, 32, 128, false)
        RT_CASE(39, float, tl::ColMajor, 192, 32, false)
        RT_CASE(40, float, tl::ColMajor, 64, 128, false)
        RT_CASE(41, float, tl::ColMajor, 96, 128, false)
        default: return -1;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

#define CRT_CASE(id, LAYOUT, R, C, SR, SC, CM)                                                      \
    case id: {                                                                                    \
        if (swizzled) {                                                                           \
            auto kern = k_chunked_roundtrip<LAYOUT<R, C>, TileShape<SR, SC>, LAYOUT<SR, SC>, true>;                                    \
            if (set_smem(kern, 140 * 1024)) return -3;                                            \
            kern<<<1, 128, 140 * 1024>>>(in, out);                                                \
        } else {                                                                                  \
            auto kern = k_chunked_roundtrip<LAYOUT<R, C>, TileShape<SR, SC>, LAYOUT<SR, SC>, false>;                                   \
            if (set_smem(kern, 140 * 1024)) return -3;                                            \
            kern<<<1, 128, 140 * 1024>>>(in, out);                                                \
        }                                                                                         \
        *rows = R; *cols = C; *col_major = CM;                                                    \
        break;                                                                                    \
    }

// 24 row-major and 13 column-major configurations: (rows, cols, shared chunk extent) of
// tests/cpp/cell/test_swizzled_copy.cu:400-429 and :433-449.
extern "C" int tcx_chunked_roundtrip_case_count() { return 37; }
extern "C" int tcx_chunked_roundtrip(int id, int swizzled, const __half* in, __half* out, int* rows, int* cols, int* col_major) {
    switch (id) {
        CRT_CASE(0, tl::RowMajor, 16, 16, 16, 16, 0)
        CRT_CASE(1, tl::RowMajor, 16, 32, 16, 32, 0)
        CRT_CASE(2, tl::RowMajor, 16, 32, 16, 32, 0)
        CRT_CASE(3, tl::RowMajor, 32, 32, 32, 32, 0)
        CRT_CASE(4, tl::RowMajor, 32, 64, 32, 32, 0)
        CRT_CASE(5, tl::RowMajor, 16, 64, 16, 32, 0)
        CRT_CASE(6, tl::RowMajor, 16, 128, 16, 64, 0)
        CRT_CASE(7, tl::RowMajor, 32, 32, 32, 32, 0)
        CRT_CASE(8, tl::RowMajor, 64, 64, 64, 64, 0)
        CRT_CASE(9, tl::RowMajor, 32, 64, 32, 32, 0)
        CRT_CASE(10, tl::RowMajor, 32, 128, 32, 64, 0)
        CRT_CASE(11, tl::RowMajor, 64, 128, 64, 64, 0)
        CRT_CASE(12, tl::RowMajor, 64, 256, 64, 128, 0)
        CRT_CASE(13, tl::RowMajor, 32, 32, 32, 32, 0)
        CRT_CASE(14, tl::RowMajor, 32, 32, 32, 32, 0)
        CRT_CASE(15, tl::RowMajor, 32, 64, 32, 32, 0)
        CRT_CASE(16, tl::RowMajor, 128, 256, 128, 128, 0)
        CRT_CASE(17, tl::RowMajor, 64, 64, 64, 64, 0)
        CRT_CASE(18, tl::RowMajor, 64, 128, 64, 64, 0)
        CRT_CASE(19, tl::RowMajor, 64, 128, 64, 128, 0)
        CRT_CASE(20, tl::RowMajor, 64, 256, 64, 128, 0)
        CRT_CASE(21, tl::RowMajor, 128, 64, 128, 64, 0)
        CRT_CASE(22, tl::RowMajor, 256, 512, 256, 256, 0)
        CRT_CASE(23, tl::RowMajor, 128, 256, 128, 128, 0)
        CRT_CASE(24, tl::ColMajor, 16, 16, 16, 16, 1)
        CRT_CASE(25, tl::ColMajor, 32, 16, 32, 16, 1)
        CRT_CASE(26, tl::ColMajor, 32, 16, 32, 16, 1)
        CRT_CASE(27, tl::ColMajor, 32, 32, 16, 32, 1)
        CRT_CASE(28, tl::ColMajor, 64, 64, 32, 64, 1)
        CRT_CASE(29, tl::ColMajor, 128, 64, 64, 64, 1)
        CRT_CASE(30, tl::ColMajor, 128, 32, 64, 32, 1)
        CRT_CASE(31, tl::ColMajor, 256, 128, 64, 128, 1)
        CRT_CASE(32, tl::ColMajor, 32, 32, 32, 32, 1)
        CRT_CASE(33, tl::ColMajor, 128, 32, 64, 32, 1)
        CRT_CASE(34, tl::ColMajor, 128, 64, 64, 64, 1)
        CRT_CASE(35, tl::ColMajor, 256, 128, 128, 128, 1)
        CRT_CASE(36, tl::ColMajor, 128, 128, 64, 128, 1)
        default: return -1;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int tcx_tile_b2b(int id, const __half* A, const __half* B, const __half* D, float* E, int* status, int* m, int* n,
                            int* k, int* p) {
    const int smem = 130 * 1024 + 1024;
    if (id == 0) {
        auto kern = k_tile_b2b<64, 64, 64, 64>;
        if (set_smem(kern, smem)) return -3;
        kern<<<1, 128, smem>>>(A, B, D, E, status);
        *m = 64; *n = 64; *k = 64; *p = 64;
    } else if (id == 1) {
        auto kern = k_tile_b2b<128, 128, 128, 128>;
        if (set_smem(kern, smem)) return -3;
        kern<<<1, 128, smem>>>(A, B, D, E, status);
        *m = 128; *n = 128; *k = 128; *p = 128;
    } else if (id == 2) {
        auto kern = k_tile_b2b<32, 128, 64, 48>;
        if (set_smem(kern, smem)) return -3;
        kern<<<1, 128, smem>>>(A, B, D, E, status);
        *m = 32; *n = 128; *k = 64; *p = 48;
    } else {
        return -1;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

#define FA_CASE(id, M, N, K, P, BN)                                                       \
    case id: {                                                                            \
        auto kern = k_tile_flash_attn<M, N, K, P, BN>;                                    \
        if (set_smem(kern, 130 * 1024 + 1024)) return -3;                                 \
        kern<<<1, 128, 130 * 1024 + 1024>>>(Q, K_, V, O, status);                         \
        *m = M; *n = N; *k = K; *p = P;                                                   \
        break;                                                                            \
    }

// The first three are the shapes the reference's attention kernel is built for (src/kernels/flash_attn.cu:438-455).
extern "C" int tcx_tile_flash_attn_case_count() { return 6; }
extern "C" int tcx_tile_flash_attn(int id, const __half* Q, const __half* K_, const __half* V, float* O, int* status, int* m,
                                   int* n, int* k, int* p) {
    switch (id) {
        FA_CASE(0, 64, 64, 128, 128, 64)
        FA_CASE(1, 64, 128, 128, 128, 64)
        FA_CASE(2, 64, 256, 128, 128, 64)
        FA_CASE(3, 128, 512, 128, 128, 128)
        FA_CASE(4, 128, 256, 64, 64, 64)
        FA_CASE(5, 32, 128, 32, 48, 32)
        default: return -1;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int tcx_row_ops(int cols, const float* in, float* softmax_out, float* row_max, float* row_sum, float* centered,
                           float* col_sum) {
    if (cols == 16)
        k_row_ops<16><<<1, 128>>>(in, softmax_out, row_max, row_sum, centered, col_sum);
    else if (cols == 64)
        k_row_ops<64><<<1, 128>>>(in, softmax_out, row_max, row_sum, centered, col_sum);
    else if (cols == 128)
        k_row_ops<128><<<1, 128>>>(in, softmax_out, row_max, row_sum, centered, col_sum);
    else
        return -1;
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
