// Tensor memory <-> registers (new on sm_100a; takes the place of the accumulator fragments that mma.sync
// leaves in registers). tcgen05.ld / st with the 32x32b shape: warp w of the CTA touches TMEM lanes
// 32*(w%4) .. +31, lane l of the warp reads or writes tile row 32*(w%4) + l, register j is column j. All
// 32 lanes of a warp must call these together (the instructions are warp-collective).
#pragma once

#include <cstdint>

#include "cell/copy/warp.hpp"
#include "types/register.hpp"
#include "types/tmem.hpp"

namespace tiledcuda::cell::copy {

namespace detail {
DEVICE void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
DEVICE void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
DEVICE uint32_t lane_quarter_base() { return static_cast<uint32_t>(((threadIdx.x >> 5) & 3) * 32) << 16; }
}  // namespace detail

// acc (TMEM, kRows x kCols fp32) -> this thread's row as RowFragment<float, kCols>. kCols % 16 == 0.
template <typename Tmem, typename Reg>
struct TmemToRegLoader {
    static_assert(Tmem::kCols == Reg::kCols && Reg::kRows == 1, "the fragment is one row of the TMEM tile");
    static_assert(Tmem::kCols % 16 == 0, "TMEM tiles are read 16 columns at a time");

    DEVICE void operator()(const Tmem& src, Reg& dst) const {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t* r = reinterpret_cast<uint32_t*>(dst.mutable_data());
#pragma unroll
        for (int c = 0; c < Tmem::kCols; c += 16) detail::tmem_ld16(src.address(c) + detail::lane_quarter_base(), r + c);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    }
};

template <typename Reg, typename Tmem>
struct RegToTmemStorer {
    static_assert(Tmem::kCols == Reg::kCols && Reg::kRows == 1, "the fragment is one row of the TMEM tile");
    static_assert(Tmem::kCols % 16 == 0, "TMEM tiles are written 16 columns at a time");

    DEVICE void operator()(const Reg& src, Tmem& dst) const {
        const uint32_t* r = reinterpret_cast<const uint32_t*>(src.data());
#pragma unroll
        for (int c = 0; c < Tmem::kCols; c += 16) detail::tmem_st16(dst.address(c) + detail::lane_quarter_base(), r + c);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
};

// TMEM allocation for a CTA: `alloc` and `free` are executed by ONE whole warp (the same one); the base
// address is written to `slot` in shared memory, to be read by everyone after a __syncthreads().
struct TmemAllocator {
    DEVICE static void alloc(uint32_t* slot, int columns) {
        const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(slot));
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s), "r"(columns) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    DEVICE static void free(uint32_t taddr, int columns) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
    }
};

}  // namespace tiledcuda::cell::copy
