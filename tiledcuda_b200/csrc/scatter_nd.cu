// scatter_nd: ScatterND assignment of slices, data[idx[t,0..k), :] = updates[t, :].
//
// Bandwidth-bound byte movement: one thread moves one 16-byte (or narrower, when alignment forces it)
// chunk of one slice. Consecutive threads read consecutive chunks of `updates` and consecutive index
// tuples, so the streamed side is fully coalesced; the scattered side writes whole 16-byte chunks.
// Each thread keeps several independent loads in flight before it stores. Offsets are 64-bit.
// Strides travel in the kernel parameters: no allocation, no host-device copy, no synchronisation.
//
// Stands in for scatter_nd_kernel / scatter_nd<T> / custom_scatter_op of the reference
// (src/kernels/scatter_nd.cu:25-50, 52-112, 114-122), which walks each slice serially with one
// atomicAdd per element; the semantics here are the assignment its test oracle checks
// (tests/python/test_scatter_nd.py:46).
#include "host.h"
#include "sm100.cuh"

namespace tcb {

constexpr int kMaxIndexRank = 8;
constexpr int kItemsPerThread = 4;
constexpr int kScatterThreads = 256;

struct ScatterShape {
    int64_t dim[kMaxIndexRank];           // extent of each indexed dimension
    int64_t slice_stride[kMaxIndexRank];  // stride of each indexed dimension, in slices
};

template <typename VecT, typename IdxT, int kK>
__global__ void __launch_bounds__(kScatterThreads)
scatter_nd_kernel(uint8_t* __restrict__ data, const uint8_t* __restrict__ updates, const IdxT* __restrict__ indices,
                  ScatterShape shape, int64_t n, int k_runtime, int64_t chunks_per_slice, uint32_t* status) {
    const int k = (kK > 0) ? kK : k_runtime;
    const int64_t total = n * chunks_per_slice;
    const int64_t base = (static_cast<int64_t>(blockIdx.x) * kItemsPerThread) * kScatterThreads + threadIdx.x;

    VecT val[kItemsPerThread];
    int64_t dst[kItemsPerThread];
    bool bad = false;

#pragma unroll
    for (int it = 0; it < kItemsPerThread; ++it) {
        const int64_t item = base + static_cast<int64_t>(it) * kScatterThreads;
        dst[it] = -1;
        if (item < total) {
            const int64_t t = (chunks_per_slice == 1) ? item : item / chunks_per_slice;
            const int64_t c = item - t * chunks_per_slice;
            int64_t slice = 0;
            bool ok = true;
#pragma unroll
            for (int j = 0; j < (kK > 0 ? kK : kMaxIndexRank); ++j) {
                if (j < k) {
                    const int64_t v = static_cast<int64_t>(__ldg(indices + t * k + j));
                    ok = ok && (v >= 0) && (v < shape.dim[j]);
                    slice += v * shape.slice_stride[j];
                }
            }
            val[it] = __ldcs(reinterpret_cast<const VecT*>(updates) + item);
            if (ok)
                dst[it] = slice * chunks_per_slice + c;
            else
                bad = true;
        }
    }
#pragma unroll
    for (int it = 0; it < kItemsPerThread; ++it) {
        if (dst[it] >= 0) reinterpret_cast<VecT*>(data)[dst[it]] = val[it];
    }
    if (bad) atomicMax(status, static_cast<uint32_t>(kDevIndexOutOfRange));
}

template <typename VecT, typename IdxT>
static int launch_scatter(void* data, const void* updates, const void* indices, const ScatterShape& shape, int64_t n,
                          int k, int64_t chunks_per_slice, uint32_t* status, cudaStream_t stream) {
    const int64_t total = n * chunks_per_slice;
    const int64_t per_block = static_cast<int64_t>(kItemsPerThread) * kScatterThreads;
    const int64_t blocks = (total + per_block - 1) / per_block;
    if (blocks > 0x7fffffffLL) return fail(TC_ERR_UNSUPPORTED, "scatter_nd: %lld chunks need too many blocks",
                                           static_cast<long long>(total));
    auto* d = static_cast<uint8_t*>(data);
    auto* u = static_cast<const uint8_t*>(updates);
    auto* i = static_cast<const IdxT*>(indices);
    const dim3 grid(static_cast<unsigned>(blocks));
    if (k == 1)
        scatter_nd_kernel<VecT, IdxT, 1><<<grid, kScatterThreads, 0, stream>>>(d, u, i, shape, n, k, chunks_per_slice,
                                                                              status);
    else if (k == 2)
        scatter_nd_kernel<VecT, IdxT, 2><<<grid, kScatterThreads, 0, stream>>>(d, u, i, shape, n, k, chunks_per_slice,
                                                                              status);
    else
        scatter_nd_kernel<VecT, IdxT, 0><<<grid, kScatterThreads, 0, stream>>>(d, u, i, shape, n, k, chunks_per_slice,
                                                                              status);
    TCB_CUDA(cudaGetLastError());
    return TC_OK;
}

template <typename VecT>
static int launch_scatter_idx(void* data, const void* updates, const void* indices, int idx_is_int64,
                              const ScatterShape& shape, int64_t n, int k, int64_t chunks_per_slice, uint32_t* status,
                              cudaStream_t stream) {
    if (idx_is_int64)
        return launch_scatter<VecT, int64_t>(data, updates, indices, shape, n, k, chunks_per_slice, status, stream);
    return launch_scatter<VecT, int32_t>(data, updates, indices, shape, n, k, chunks_per_slice, status, stream);
}

// ---------------------------------------------------------------------------------------------------
// Accumulating variant: data[idx[t,0..k), :] += updates[t, :]; repeated tuples add up. One thread owns one
// 16-byte chunk of one slice when pointers and slice size allow it, else one element, and issues one
// reduction (vector red.global.add where the type has one) without reading the table back.
enum ScatterAddType { kAddF32 = 0, kAddF16 = 1, kAddI32 = 2, kAddF64 = 3 };

template <int kType, bool kVec>
struct AddChunk;
template <>
struct AddChunk<kAddF32, true> {
    using T = float4;
    static __device__ __forceinline__ void add(T* p, T v) { atomicAdd(p, v); }
};
template <>
struct AddChunk<kAddF32, false> {
    using T = float;
    static __device__ __forceinline__ void add(T* p, T v) { atomicAdd(p, v); }
};
template <>
struct AddChunk<kAddF16, true> {
    using T = uint4;   // eight halves: four packed-pair reductions
    static __device__ __forceinline__ void add(T* p, T v) {
        __half2* d = reinterpret_cast<__half2*>(p);
        const __half2* s = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) atomicAdd(d + i, s[i]);
    }
};
template <>
struct AddChunk<kAddF16, false> {
    using T = __half;
    static __device__ __forceinline__ void add(T* p, T v) { atomicAdd(p, v); }
};
template <>
struct AddChunk<kAddI32, true> {
    using T = int4;
    static __device__ __forceinline__ void add(T* p, T v) {
        int* d = reinterpret_cast<int*>(p);
        atomicAdd(d, v.x);
        atomicAdd(d + 1, v.y);
        atomicAdd(d + 2, v.z);
        atomicAdd(d + 3, v.w);
    }
};
template <>
struct AddChunk<kAddI32, false> {
    using T = int;
    static __device__ __forceinline__ void add(T* p, T v) { atomicAdd(p, v); }
};
template <>
struct AddChunk<kAddF64, true> {
    using T = double2;
    static __device__ __forceinline__ void add(T* p, T v) {
        double* d = reinterpret_cast<double*>(p);
        atomicAdd(d, v.x);
        atomicAdd(d + 1, v.y);
    }
};
template <>
struct AddChunk<kAddF64, false> {
    using T = double;
    static __device__ __forceinline__ void add(T* p, T v) { atomicAdd(p, v); }
};

template <int kType, bool kVec, typename IdxT>
__global__ void __launch_bounds__(kScatterThreads)
scatter_nd_add_kernel(uint8_t* __restrict__ data, const uint8_t* __restrict__ updates, const IdxT* __restrict__ indices,
                      ScatterShape shape, int64_t n, int k, int64_t chunks_per_slice, uint32_t* status) {
    using Op = AddChunk<kType, kVec>;
    using T = typename Op::T;
    const int64_t total = n * chunks_per_slice;
    const int64_t base = (static_cast<int64_t>(blockIdx.x) * kItemsPerThread) * kScatterThreads + threadIdx.x;
    T val[kItemsPerThread];
    int64_t dst[kItemsPerThread];
    bool bad = false;
#pragma unroll
    for (int it = 0; it < kItemsPerThread; ++it) {
        const int64_t item = base + static_cast<int64_t>(it) * kScatterThreads;
        dst[it] = -1;
        if (item < total) {
            const int64_t t = (chunks_per_slice == 1) ? item : item / chunks_per_slice;
            const int64_t c = item - t * chunks_per_slice;
            int64_t slice = 0;
            bool ok = true;
            for (int j = 0; j < k; ++j) {
                const int64_t v = static_cast<int64_t>(__ldg(indices + t * k + j));
                ok = ok && (v >= 0) && (v < shape.dim[j]);
                slice += v * shape.slice_stride[j];
            }
            val[it] = reinterpret_cast<const T*>(updates)[item];
            if (ok)
                dst[it] = slice * chunks_per_slice + c;
            else
                bad = true;
        }
    }
#pragma unroll
    for (int it = 0; it < kItemsPerThread; ++it) {
        if (dst[it] >= 0) Op::add(reinterpret_cast<T*>(data) + dst[it], val[it]);
    }
    if (bad) atomicMax(status, static_cast<uint32_t>(kDevIndexOutOfRange));
}

template <int kType, bool kVec>
static int launch_scatter_add(void* data, const void* updates, const void* indices, int idx_is_int64,
                              const ScatterShape& shape, int64_t n, int k, int64_t chunks_per_slice, uint32_t* status,
                              cudaStream_t stream) {
    const int64_t total = n * chunks_per_slice;
    const int64_t per_block = static_cast<int64_t>(kItemsPerThread) * kScatterThreads;
    const int64_t blocks = (total + per_block - 1) / per_block;
    if (blocks > 0x7fffffffLL) return fail(TC_ERR_UNSUPPORTED, "scatter_nd_add: %lld chunks need too many blocks",
                                           static_cast<long long>(total));
    auto* d = static_cast<uint8_t*>(data);
    auto* u = static_cast<const uint8_t*>(updates);
    const dim3 grid(static_cast<unsigned>(blocks));
    if (idx_is_int64)
        scatter_nd_add_kernel<kType, kVec, int64_t><<<grid, kScatterThreads, 0, stream>>>(
            d, u, static_cast<const int64_t*>(indices), shape, n, k, chunks_per_slice, status);
    else
        scatter_nd_add_kernel<kType, kVec, int32_t><<<grid, kScatterThreads, 0, stream>>>(
            d, u, static_cast<const int32_t*>(indices), shape, n, k, chunks_per_slice, status);
    TCB_CUDA(cudaGetLastError());
    return TC_OK;
}

template <int kType>
static int scatter_add_typed(void* data, const void* updates, const void* indices, int idx_is_int64,
                             const ScatterShape& shape, int64_t n, int k, int64_t slice_elems, int elem_bytes,
                             uint32_t* status, cudaStream_t stream) {
    const int64_t slice_bytes = slice_elems * elem_bytes;
    const uintptr_t align_bits =
        reinterpret_cast<uintptr_t>(data) | reinterpret_cast<uintptr_t>(updates) | static_cast<uintptr_t>(slice_bytes);
    if ((align_bits & 15u) == 0)
        return launch_scatter_add<kType, true>(data, updates, indices, idx_is_int64, shape, n, k, slice_bytes / 16, status,
                                               stream);
    return launch_scatter_add<kType, false>(data, updates, indices, idx_is_int64, shape, n, k, slice_elems, status, stream);
}

// Validates the arguments shared by both entry points and fills the indexed-dimension strides.
static int scatter_shape(const char* op, const void* data, const void* updates, const void* indices, const int64_t* dims,
                         int rank, int64_t n, int k, ScatterShape* shape, int64_t* slice_elems) {
    TCB_REQUIRE(data && dims, "%s: null pointer argument", op);
    TCB_REQUIRE(n <= 0 || (updates && indices), "%s: null pointer argument", op);
    TCB_REQUIRE(rank >= 1 && rank <= 16, "%s: rank %d outside [1,16]", op, rank);
    TCB_REQUIRE(k >= 1 && k <= rank && k <= kMaxIndexRank, "%s: index tuple length %d outside [1,min(rank,%d)]", op, k,
                kMaxIndexRank);
    TCB_REQUIRE(n >= 0, "%s: negative n", op);
    for (int i = 0; i < rank; ++i) TCB_REQUIRE(dims[i] > 0, "%s: dims[%d] = %lld", op, i, (long long)dims[i]);
    *slice_elems = 1;
    for (int i = k; i < rank; ++i) *slice_elems *= dims[i];
    int64_t stride = 1;
    for (int j = k - 1; j >= 0; --j) {
        shape->dim[j] = dims[j];
        shape->slice_stride[j] = stride;
        stride *= dims[j];
    }
    return TC_OK;
}

}  // namespace tcb

extern "C" int tc_scatter_nd(void* data, const void* updates, const void* indices, int idx_is_int64,
                             const int64_t* dims, int rank, int64_t n, int k, int elem_bytes, tc_stream_t stream) {
    using namespace tcb;
    TCB_REQUIRE(data && dims, "scatter_nd: null pointer argument");
    TCB_REQUIRE(n <= 0 || (updates && indices), "scatter_nd: null pointer argument");
    TCB_REQUIRE(rank >= 1 && rank <= 16, "scatter_nd: rank %d outside [1,16]", rank);
    TCB_REQUIRE(k >= 1 && k <= rank && k <= kMaxIndexRank, "scatter_nd: index tuple length %d outside [1,min(rank,%d)]",
                k, kMaxIndexRank);
    TCB_REQUIRE(elem_bytes == 1 || elem_bytes == 2 || elem_bytes == 4 || elem_bytes == 8,
                "scatter_nd: elem_bytes %d not in {1,2,4,8}", elem_bytes);
    TCB_REQUIRE(n >= 0, "scatter_nd: negative n");
    for (int i = 0; i < rank; ++i) TCB_REQUIRE(dims[i] > 0, "scatter_nd: dims[%d] = %lld", i, (long long)dims[i]);
    if (n == 0) return TC_OK;

    const DeviceInfo* dev = nullptr;
    if (int rc = current_device(&dev)) return rc;

    ScatterShape shape{};
    int64_t slice_elems = 1;
    for (int i = k; i < rank; ++i) slice_elems *= dims[i];
    int64_t stride = 1;
    for (int j = k - 1; j >= 0; --j) {
        shape.dim[j] = dims[j];
        shape.slice_stride[j] = stride;
        stride *= dims[j];
    }
    const int64_t slice_bytes = slice_elems * elem_bytes;
    const uintptr_t align_bits =
        reinterpret_cast<uintptr_t>(data) | reinterpret_cast<uintptr_t>(updates) | static_cast<uintptr_t>(slice_bytes);
    auto* st = static_cast<cudaStream_t>(stream);

    if ((align_bits & 15u) == 0)
        return launch_scatter_idx<uint4>(data, updates, indices, idx_is_int64, shape, n, k, slice_bytes / 16,
                                         dev->status_word, st);
    if ((align_bits & 7u) == 0)
        return launch_scatter_idx<uint2>(data, updates, indices, idx_is_int64, shape, n, k, slice_bytes / 8,
                                         dev->status_word, st);
    if ((align_bits & 3u) == 0)
        return launch_scatter_idx<uint32_t>(data, updates, indices, idx_is_int64, shape, n, k, slice_bytes / 4,
                                            dev->status_word, st);
    if ((align_bits & 1u) == 0)
        return launch_scatter_idx<uint16_t>(data, updates, indices, idx_is_int64, shape, n, k, slice_bytes / 2,
                                            dev->status_word, st);
    return launch_scatter_idx<uint8_t>(data, updates, indices, idx_is_int64, shape, n, k, slice_bytes,
                                       dev->status_word, st);
}

extern "C" int tc_scatter_nd_add(void* data, const void* updates, const void* indices, int idx_is_int64,
                                 const int64_t* dims, int rank, int64_t n, int k, int elem_type, tc_stream_t stream) {
    using namespace tcb;
    ScatterShape shape{};
    int64_t slice_elems = 0;
    if (int rc = scatter_shape("scatter_nd_add", data, updates, indices, dims, rank, n, k, &shape, &slice_elems)) return rc;
    TCB_REQUIRE(elem_type >= kAddF32 && elem_type <= kAddF64, "scatter_nd_add: elem_type %d not in {0: f32, 1: f16, 2: i32, 3: f64}",
                elem_type);
    const int elem_bytes = elem_type == kAddF16 ? 2 : (elem_type == kAddF64 ? 8 : 4);
    TCB_REQUIRE(((reinterpret_cast<uintptr_t>(data) | reinterpret_cast<uintptr_t>(updates)) & (elem_bytes - 1)) == 0,
                "scatter_nd_add: data and updates must be aligned to the element size");
    if (n == 0) return TC_OK;
    const DeviceInfo* dev = nullptr;
    if (int rc = current_device(&dev)) return rc;
    auto* st = static_cast<cudaStream_t>(stream);
    switch (elem_type) {
        case kAddF32:
            return scatter_add_typed<kAddF32>(data, updates, indices, idx_is_int64, shape, n, k, slice_elems, 4, dev->status_word, st);
        case kAddF16:
            return scatter_add_typed<kAddF16>(data, updates, indices, idx_is_int64, shape, n, k, slice_elems, 2, dev->status_word, st);
        case kAddI32:
            return scatter_add_typed<kAddI32>(data, updates, indices, idx_is_int64, shape, n, k, slice_elems, 4, dev->status_word, st);
        default:
            return scatter_add_typed<kAddF64>(data, updates, indices, idx_is_int64, shape, n, k, slice_elems, 8, dev->status_word, st);
    }
}
