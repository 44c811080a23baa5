// Host-side plumbing: error text, device cache, tensor-map encoding, device status word.
#include "host.h"

#include <mutex>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

namespace tcb {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

static constexpr int kMaxDevices = 64;
static DeviceInfo g_dev[kMaxDevices];
static bool g_dev_ready[kMaxDevices];
static std::mutex g_mu;

int current_device(const DeviceInfo** out) {
    int dev = -1;
    TCB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(TC_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_dev_ready[dev]) {
        DeviceInfo d;
        d.device = dev;
        TCB_CUDA(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
        TCB_CUDA(cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
        TCB_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
        TCB_CUDA(cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        if (d.cc_major != 10)
            return fail(TC_ERR_UNSUPPORTED, "device %d is sm_%d%d; these kernels are built for sm_100a only", dev,
                        d.cc_major, d.cc_minor);
        TCB_CUDA(cudaMalloc(reinterpret_cast<void**>(&d.status_word), 4 * sizeof(uint32_t)));
        TCB_CUDA(cudaMemset(d.status_word, 0, 4 * sizeof(uint32_t)));
        g_dev[dev] = d;
        g_dev_ready[dev] = true;
    }
    *out = &g_dev[dev];
    return TC_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn g_encode = nullptr;

static int load_encode() {
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_encode) return TC_OK;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    TCB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || fn == nullptr)
        return fail(TC_ERR_CUDA, "driver has no cuTensorMapEncodeTiled (query result %d)", static_cast<int>(qres));
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    return TC_OK;
}

int encode_tmap_f16_sw128(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                          const uint64_t* strides_bytes, const uint32_t* box, bool bf16) {
    if (int rc = load_encode()) return rc;
    cuuint64_t gdim[5];
    cuuint64_t gstride[5];
    cuuint32_t bdim[5];
    cuuint32_t estride[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bdim[i] = box[i];
        estride[i] = 1;
        if (i + 1 < rank) gstride[i] = strides_bytes[i];
    }
    CUresult r = g_encode(out, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, static_cast<cuuint32_t>(rank),
                          const_cast<void*>(base), gdim, gstride, bdim, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(TC_ERR_CUDA,
                    "cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims %llu x %llu, box %u x %u)",
                    static_cast<int>(r), rank, (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 1),
                    box[0], rank > 1 ? box[1] : 1u);
    return TC_OK;
}

int encode_tmap_f32_sw128(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t row_stride_bytes,
                          uint32_t box_cols, uint32_t box_rows) {
    if (int rc = load_encode()) return rc;
    const cuuint64_t gdim[2] = {cols, rows};
    const cuuint64_t gstride[1] = {row_stride_bytes};
    const cuuint32_t bdim[2] = {box_cols, box_rows};
    const cuuint32_t estride[2] = {1, 1};
    CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), gdim, gstride, bdim, estride,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(TC_ERR_CUDA, "cuTensorMapEncodeTiled (fp32 output) failed with CUresult %d (%llu x %llu, stride %llu)",
                    static_cast<int>(r), (unsigned long long)cols, (unsigned long long)rows,
                    (unsigned long long)row_stride_bytes);
    return TC_OK;
}

int encode_tmap_f32_sw128_3d(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t batch,
                             uint32_t box_cols, uint32_t box_rows) {
    if (int rc = load_encode()) return rc;
    const cuuint64_t gdim[3] = {cols, rows, batch};
    const cuuint64_t gstride[2] = {cols * 4, rows * cols * 4};
    const cuuint32_t bdim[3] = {box_cols, box_rows, 1};
    const cuuint32_t estride[3] = {1, 1, 1};
    CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), gdim, gstride, bdim, estride,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(TC_ERR_CUDA, "cuTensorMapEncodeTiled (fp32 output, 3-D) failed with CUresult %d (%llu x %llu x %llu)",
                    static_cast<int>(r), (unsigned long long)cols, (unsigned long long)rows, (unsigned long long)batch);
    return TC_OK;
}

}  // namespace tcb

extern "C" {

const char* tc_last_error(void) { return tcb::g_err; }

int tc_version(void) { return 1000; }

int tc_device_status(int* code) {
    if (code == nullptr) return tcb::fail(TC_ERR_BAD_ARG, "tc_device_status: code is NULL");
    const tcb::DeviceInfo* dev = nullptr;
    if (int rc = tcb::current_device(&dev)) return rc;
    uint32_t host_word = 0;
    TCB_CUDA(cudaDeviceSynchronize());
    TCB_CUDA(cudaMemcpy(&host_word, dev->status_word, sizeof(host_word), cudaMemcpyDeviceToHost));
    if (host_word != 0) TCB_CUDA(cudaMemset(dev->status_word, 0, 4 * sizeof(uint32_t)));
    *code = static_cast<int>(host_word);
    return TC_OK;
}

// ---- peer windows: another rank's device buffer, addressable from this process -------------------------------
// One process per GPU. A rank exports a device allocation (cudaIpcGetMemHandle wants a pointer into a cudaMalloc
// allocation and names the whole allocation), the others open it with the device they compute on current, which
// maps it into THEIR context with peer access to the owner's GPU. A copy from local memory into such a window is a
// device-to-device cudaMemcpyAsync over NVLink, executed by the copy engines.
int tc_peer_export(const void* dev_ptr, void* handle_out, int64_t handle_bytes) {
    using namespace tcb;
    TCB_REQUIRE(dev_ptr != nullptr && handle_out != nullptr, "peer_export: null pointer argument");
    TCB_REQUIRE(handle_bytes >= static_cast<int64_t>(sizeof(cudaIpcMemHandle_t)), "peer_export: the handle buffer holds %lld bytes, %zu needed",
                (long long)handle_bytes, sizeof(cudaIpcMemHandle_t));
    cudaIpcMemHandle_t h;
    TCB_CUDA(cudaIpcGetMemHandle(&h, const_cast<void*>(dev_ptr)));
    memcpy(handle_out, &h, sizeof(h));
    return TC_OK;
}

int tc_peer_open(const void* handle, int64_t handle_bytes, void** base_out) {
    using namespace tcb;
    TCB_REQUIRE(handle != nullptr && base_out != nullptr, "peer_open: null pointer argument");
    TCB_REQUIRE(handle_bytes >= static_cast<int64_t>(sizeof(cudaIpcMemHandle_t)), "peer_open: the handle buffer holds %lld bytes, %zu needed",
                (long long)handle_bytes, sizeof(cudaIpcMemHandle_t));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    TCB_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *base_out = p;
    return TC_OK;
}

int tc_peer_close(void* base) {
    using namespace tcb;
    if (base == nullptr) return TC_OK;
    TCB_CUDA(cudaIpcCloseMemHandle(base));
    return TC_OK;
}

int tc_peer_copy(void* dst, const void* src, int64_t bytes, tc_stream_t stream) {
    using namespace tcb;
    TCB_REQUIRE(dst != nullptr && src != nullptr && bytes >= 0, "peer_copy: null pointer or negative size");
    if (bytes == 0) return TC_OK;
    TCB_CUDA(cudaMemcpyAsync(dst, src, static_cast<size_t>(bytes), cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
    return TC_OK;
}

}  // extern "C"
