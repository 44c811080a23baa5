// C entry point around the reference's own host flash attention oracle `host_flash_attn`
// (examples/cpp/03_flash_attention/flash_attn_cpu.hpp:9-100), compiled from where it lies in the
// reference tree. TEST INFRASTRUCTURE ONLY. It allocates the scratch vectors the reference's
// driver allocates (examples/cpp/03_flash_attention/flash_attn.cu) and zero-fills them and O.
#include <cuda_fp16.h>

#include <vector>

#include "flash_attn_cpu.hpp"

extern "C" void ref_host_flash_attn(int m, int n, int k, int p, const __half* q, const __half* kmat, const __half* v,
                                    __half* o) {
    const __half zero = __float2half(0.f);
    std::vector<__half> acc(static_cast<size_t>(m) * n, zero), exp_values(static_cast<size_t>(m) * p, zero);
    std::vector<__half> cur_row_max(m, zero), prev_row_max(m, zero), new_row_max(m, zero), prev_norm(m, zero),
        new_norm(m, zero), prev_sums(m, zero), cur_sums(m, zero), new_sums(m, zero);
    for (int i = 0; i < m * p; ++i) o[i] = zero;
    host_flash_attn(m, n, k, p, /*kBatch=*/1, q, kmat, v, o, acc.data(), exp_values.data(), cur_row_max.data(),
                    prev_row_max.data(), new_row_max.data(), prev_norm.data(), new_norm.data(), prev_sums.data(),
                    cur_sums.data(), new_sums.data());
}
