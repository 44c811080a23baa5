// Tile matrix multiply-accumulate on the 5th-generation tensor cores.
//
//   gemm(a, b, acc, accumulate)     acc[M, N] (+)= a[M, K] * b[K, N]
//
// a is a 16-bit SharedTile in operand layout with M = kOuter <= 128 rows; b is a 16-bit SharedTile whose
// operand view has N = kOuter (a ColMajor<K, N> tile as in the reference, or a RowMajor<N, K> tile); acc is
// a TmemTile<float, RowMajor<128 or M, N>>. One thread (thread 0 of the CTA) issues K/16 tcgen05.mma
// instructions (kind::f16: fp16 inputs, fp32 accumulation, the only mode the reference's gemm has either:
// include/cell/compute/gemm.hpp:26-35); every thread may call it. The instruction always computes 128
// rows: rows beyond M read whatever follows the tile in shared memory and land in TMEM lanes >= M, which
// nobody reads, so a's storage must be followed by enough valid shared memory for 128 rows.
// The MMAs are asynchronous: commit an MmaBarrier after the call and wait on it before reading acc or
// overwriting a / b.
#pragma once

#include <cstdint>

#include "cell/copy/shared_to_register.hpp"
#include "cell/sync.hpp"
#include "types/shared.hpp"
#include "types/tmem.hpp"

namespace tiledcuda::cell::compute {

namespace detail {
// kind::f16 instruction descriptor: D fp32, A/B fp16, both K-major, N/8 at bit 17, M/16 at bit 24.
HOST_DEVICE constexpr uint32_t instr_desc_f16(int m, int n) {
    return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

DEVICE void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate))
        : "memory");
}
}  // namespace detail

template <typename SharedA, typename SharedB, typename TmemC>
DEVICE void gemm(const SharedA& a, const SharedB& b, TmemC& acc, bool accumulate = true) {
    static_assert(SharedA::kIsOperand && SharedB::kIsOperand, "operands must be 16-bit shared tiles");
    static_assert(SharedA::kK == SharedB::kK, "the contraction lengths of a and b differ");
    static_assert(SharedA::kK % 16 == 0, "K must be a multiple of 16");
    static_assert(SharedA::kOuter <= 128, "one CTA accumulates at most 128 rows");
    static_assert(SharedB::kOuter % 16 == 0 && SharedB::kOuter <= 256, "N must be a multiple of 16, at most 256");
    static_assert(TmemC::kCols == SharedB::kOuter, "accumulator width must equal N");
    if (threadIdx.x == 0) {
        constexpr uint32_t idesc = detail::instr_desc_f16(128, SharedB::kOuter);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int k = 0; k < SharedA::kK / 16; ++k)
            detail::mma_f16_ss(acc.address(), copy::make_operand_descriptor(a, k), copy::make_operand_descriptor(b, k), idesc,
                               accumulate || k > 0);
    }
}

}  // namespace tiledcuda::cell::compute
