// CTA-cooperative copies between global and shared memory.
//
// GlobalToSharedLoader<Shared, WarpLayout>: every thread of the CTA moves 16-byte pieces with cp.async
// (coalesced on the global side) and places each piece where the Shared tile's layout puts it, i.e. in
// the 128-byte-swizzled or interleaved operand layout tcgen05.mma reads. The copy is asynchronous: finish
// it with __copy_async() and __syncthreads(), as with the reference's loader
// (include/cell/copy/global_to_shared.hpp:250-289). SharedToGlobalStorer is the inverse, synchronous.
// TmaTileLoader is the tensor-map route (one thread, one instruction per 64-column chunk) for kernels
// whose host side built a CUtensorMap; it needs the swizzled layout.
#pragma once

#include <cstdint>
#if defined(__CUDACC__)
#include <cuda.h>
#endif

#include "cell/copy/warp.hpp"
#include "types/global.hpp"
#include "types/shared.hpp"

namespace tiledcuda::cell::copy {

namespace detail {
DEVICE void cp_async_16(void* smem_dst, const void* gmem_src) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem_src) : "memory");
}
}  // namespace detail

template <typename Shared_, typename WarpLayout_>
struct GlobalToSharedLoader : warp::CopyBase<WarpLayout_> {
    using Shared = Shared_;
    using DType = typename Shared::DType;
    using Base = warp::CopyBase<WarpLayout_>;
    static constexpr int kPerPiece = 16 / static_cast<int>(sizeof(DType));  // elements per 16-byte piece

    template <typename Global>
    DEVICE void operator()(const Global& src, Shared& dst) const {
        static_assert(Global::kRows == Shared::kRows && Global::kCols == Shared::kCols, "tile shapes differ");
        static_assert(Global::kType == Shared::kType, "source and destination must have the same majorness");
        constexpr bool kRowMajor = Shared::kType == tl::Layout::kRowMajor;
        constexpr int kOuter = kRowMajor ? Shared::kRows : Shared::kCols;   // strided extent
        constexpr int kInner = kRowMajor ? Shared::kCols : Shared::kRows;   // contiguous extent
        static_assert(kInner % kPerPiece == 0, "the contiguous extent must be a multiple of 16 bytes");
        constexpr int kPiecesPerLine = kInner / kPerPiece;
        constexpr int kPieces = kOuter * kPiecesPerLine;
        DType* sdata = dst.mutable_data();
        for (int p = static_cast<int>(threadIdx.x); p < kPieces; p += Base::kThreads) {
            const int o = p / kPiecesPerLine;
            const int i = (p - o * kPiecesPerLine) * kPerPiece;
            const int x = kRowMajor ? o : i;
            const int y = kRowMajor ? i : o;
            detail::cp_async_16(sdata + Shared::offset(x, y), &src(x, y));
        }
    }
};

template <typename Shared_, typename WarpLayout_>
struct SharedToGlobalStorer : warp::CopyBase<WarpLayout_> {
    using Shared = Shared_;
    using DType = typename Shared::DType;
    using Base = warp::CopyBase<WarpLayout_>;
    static constexpr int kPerPiece = 16 / static_cast<int>(sizeof(DType));

    template <typename Global>
    DEVICE void operator()(const Shared& src, Global& dst) const {
        static_assert(Global::kRows == Shared::kRows && Global::kCols == Shared::kCols, "tile shapes differ");
        static_assert(Global::kType == Shared::kType, "source and destination must have the same majorness");
        constexpr bool kRowMajor = Shared::kType == tl::Layout::kRowMajor;
        constexpr int kOuter = kRowMajor ? Shared::kRows : Shared::kCols;
        constexpr int kInner = kRowMajor ? Shared::kCols : Shared::kRows;
        static_assert(kInner % kPerPiece == 0, "the contiguous extent must be a multiple of 16 bytes");
        constexpr int kPiecesPerLine = kInner / kPerPiece;
        constexpr int kPieces = kOuter * kPiecesPerLine;
        const DType* sdata = src.data();
        for (int p = static_cast<int>(threadIdx.x); p < kPieces; p += Base::kThreads) {
            const int o = p / kPiecesPerLine;
            const int i = (p - o * kPiecesPerLine) * kPerPiece;
            const int x = kRowMajor ? o : i;
            const int y = kRowMajor ? i : o;
            *reinterpret_cast<uint4*>(&dst(x, y)) = *reinterpret_cast<const uint4*>(sdata + Shared::offset(x, y));
        }
    }
};

#if defined(__CUDACC__)
// Tensor-map load of a swizzled 16-bit operand tile: one cp.async.bulk.tensor per 64-element K chunk,
// issued by ONE thread; completion is counted in bytes on `mbar` (the caller arms it with
// Shared::kBytes). `k0` / `outer0` are the element coordinates of the tile in the tensor.
template <typename Shared_>
struct TmaTileLoader {
    using Shared = Shared_;
    static_assert(Shared::kIsOperand && Shared::kSwizzled, "TMA tiles use the 128-byte swizzled operand layout");

    DEVICE void operator()(const CUtensorMap* map, Shared& dst, uint64_t* mbar, int k0, int outer0) const {
        using Op = typename Shared::Operand;
        const uint32_t bar = static_cast<uint32_t>(__cvta_generic_to_shared(mbar));
        for (int c = 0; c < Op::kChunks; ++c) {
            const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst.mutable_data())) + c * Op::kChunkBytes;
            asm volatile(
                "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                ::"r"(d), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(k0 + c * Op::kChunkElems), "r"(outer0)
                : "memory");
        }
    }
};
#endif

}  // namespace tiledcuda::cell::copy
