// Host-side plumbing shared by the launchers: thread-local error text, CUDA call checking that
// returns a status instead of exiting, TMA tensor-map encoding through the runtime's driver entry
// point (so the library carries no link-time dependency on libcuda), device properties and the
// per-device status word that kernels write on a bounded-wait timeout.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/tiledcuda_b200.h"

namespace tcb {

// printf-style; stores the message for tc_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);

#define TCB_CUDA(expr)                                                                            \
    do {                                                                                          \
        cudaError_t _e = (expr);                                                                  \
        if (_e != cudaSuccess)                                                                    \
            return ::tcb::fail(TC_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                               __FILE__, __LINE__);                                               \
    } while (0)

#define TCB_REQUIRE(cond, ...)                                      \
    do {                                                            \
        if (!(cond)) return ::tcb::fail(TC_ERR_BAD_ARG, __VA_ARGS__); \
    } while (0)

struct DeviceInfo {
    int device = -1;
    int cc_major = 0;
    int cc_minor = 0;
    int sm_count = 0;
    int max_smem_optin = 0;
    uint32_t* status_word = nullptr;  // device memory, 4 words, zero-initialised
};

// Info for the current device (cached; thread-safe). Fails with TC_ERR_UNSUPPORTED unless sm_100.
int current_device(const DeviceInfo** out);

// Encodes a tiled fp16 tensor map with 128-byte swizzle. dims/box are innermost-first; strides_bytes has
// rank-1 entries (stride of dims 1..rank-1). Zero fill outside the tensor.
int encode_tmap_f16_sw128(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                          const uint64_t* strides_bytes, const uint32_t* box, bool bf16 = false);

// Tiled fp32 2-D map with 128-byte swizzle (rows of 32 floats), for TMA stores of accumulator tiles.
int encode_tmap_f32_sw128(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t row_stride_bytes,
                          uint32_t box_cols, uint32_t box_rows);

// The same for a [batch, rows, cols] fp32 array (cols innermost, dense): boxes of box_cols x box_rows x 1.
int encode_tmap_f32_sw128_3d(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t batch,
                             uint32_t box_cols, uint32_t box_rows);

// One-time, per-device set-up of a kernel (its dynamic shared-memory limit), safe against concurrent first calls
// from several host threads: every launcher keeps one of these per kernel and calls raise_smem_limit_once() with it.
struct OncePerDevice {
    std::mutex mu;
    bool done[64] = {};
};

template <typename Kernel>
inline int raise_smem_limit_once(OncePerDevice& once, int device, Kernel kernel, int bytes) {
    if (device < 0 || device >= 64) return fail(TC_ERR_UNSUPPORTED, "device ordinal %d out of range", device);
    std::lock_guard<std::mutex> lock(once.mu);
    if (!once.done[device]) {
        TCB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
        once.done[device] = true;
    }
    return TC_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Launch with programmatic stream serialization: if the kernel before it in the stream releases its dependents
// early (griddepcontrol.launch_dependents), this kernel's CTAs may start on free SMs and run their set-up while
// that kernel drains. The kernel must execute griddepcontrol.wait before it touches global memory; behind a kernel
// that never releases early the launch behaves like a plain one.
template <typename... Params, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

}  // namespace tcb
