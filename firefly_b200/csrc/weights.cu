// Getting weights onto the device: a pinned mapping of the checkpoint file, asynchronous copies
// straight into their final place in one device arena, conversion of the element type on the
// device, and seeded random weights whose values are the same bits on the CPU and on the GPU.
//
// The reference maps the file and registers the mapping with the driver as read-only host
// memory, falling back to pageable memory without a word when that fails
// (include/firefly/mm/memory_mapper.h:117-135), sizes one device chunk in a first pass and
// bump-allocates every tensor in it at 256-byte alignment (include/firefly/model_loader.h:48-58,
// include/firefly/mm/model_weight_pool.h:58-109), and then copies tensor by tensor with a blocking
// cudaMemcpy, converting BF16 to FP16 element by element on the host (model_loader.h:79-108).
// Here the copies are asynchronous on the caller's stream, rows can be scattered into a fused
// matrix (q|k|v stacked, gate and up interleaved in groups of rows) by one strided copy per
// source tensor, and a tensor whose stored type is not the device type passes through a staging
// buffer on the device and a conversion kernel.
//
// Row placement, shared by the copy, the conversion and the random kernels: source row r of a
// tensor with `rows` rows goes to destination row  dst_row0 + (r / group) * group_stride + r % group.
// group == rows (and any stride) is a plain block of rows.
#include "common.cuh"

#include <cuda_fp16.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace ff {

struct MappedFile {
    void* addr;
    size_t size;
    int pinned;      // 1: registered with the driver (copies from it are asynchronous)
};

enum : int { WT_F32 = 0, WT_BF16 = 1, WT_F16 = 2, WT_F64 = 3 };

template <typename T> __device__ __forceinline__ float wt_load(const T* p, size_t i);
template <> __device__ __forceinline__ float wt_load<float>(const float* p, size_t i) { return p[i]; }
template <> __device__ __forceinline__ float wt_load<bf16>(const bf16* p, size_t i) { return __bfloat162float(p[i]); }
template <> __device__ __forceinline__ float wt_load<__half>(const __half* p, size_t i) { return __half2float(p[i]); }
template <> __device__ __forceinline__ float wt_load<double>(const double* p, size_t i) { return (float)p[i]; }

// dst[placed row][c] = convert(src[r][c]); one thread per element, rows of `cols` elements
template <typename TS, typename TD>
__global__ void convert_rows_kernel(const TS* __restrict__ src, TD* __restrict__ dst, long long rows, long long cols,
                                    long long dst_row0, long long group, long long group_stride) {
    const long long n = rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cols, c = i - r * cols;
        const long long dr = dst_row0 + (r / group) * group_stride + r % group;
        dst[dr * cols + c] = from_float<TD>(wt_load<TS>(src, (size_t)i));
    }
}

// --------------------------------------------------------------------------------------------
// Seeded random values, the same bits wherever they are computed: only integer arithmetic and
// single correctly rounded float operations are used.
//   h      = mix64(key + index * 0x9E3779B97F4A7C15)        index: element's place in its *source* tensor
//   u      = h >> 32;  knot = u >> 16;  frac = u & 0xffff
//   fixed  = table[knot] + (((table[knot+1] - table[knot]) * frac) >> 16)     table: quantiles of N(0,1) in units of 2^-24
//   value  = float(fixed) * scale + shift                   (one rounding each: conversion, product, sum)
// The table (65537 int32 knots) is made once on the host in 64-bit floating point and handed to
// both implementations.  Integer tensors: h % high.
__device__ __forceinline__ float random_normal_value(uint64_t key, uint64_t index, const int* __restrict__ table,
                                                     float scale, float shift) {
    const uint64_t h = mix64(key + index * 0x9E3779B97F4A7C15ull);
    const uint32_t u = (uint32_t)(h >> 32);
    const int knot = (int)(u >> 16);
    const long long frac = (long long)(u & 0xffffu);
    const long long t0 = table[knot], t1 = table[knot + 1];
    const long long fixed = t0 + (((t1 - t0) * frac) >> 16);
    return __fadd_rn(__fmul_rn(__ll2float_rn(fixed), scale), shift);
}

// via_bf16: the value is first rounded to bfloat16, the type a checkpoint of this model would store
// it in, and then widened (a tensor that is kept in 32-bit on the device, like a norm weight)
template <typename TD>
__global__ void random_rows_kernel(TD* __restrict__ dst, long long rows, long long cols, long long dst_row0,
                                   long long group, long long group_stride, uint64_t key,
                                   const int* __restrict__ table, float scale, float shift, int via_bf16) {
    const long long n = rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cols, c = i - r * cols;
        const long long dr = dst_row0 + (r / group) * group_stride + r % group;
        float v = random_normal_value(key, (uint64_t)i, table, scale, shift);
        if (via_bf16) v = __bfloat162float(__float2bfloat16_rn(v));
        dst[dr * cols + c] = from_float<TD>(v);
    }
}

__global__ void random_int_rows_kernel(int* __restrict__ dst, long long n, uint64_t key, unsigned long long high) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dst[i] = (int)(mix64(key + (uint64_t)i * 0x9E3779B97F4A7C15ull) % high);
}

// blocks of 256 threads for n elements; the kernels stride over what a capped grid leaves
static inline int grid_for(long long n) {
    const long long g = (n + 255) / 256;
    return (int)(g < 1 ? 1 : (g > 4096 ? 4096 : g));
}

template <typename TS>
static int convert_dispatch(const void* src, void* dst, int dst_type, long long rows, long long cols, long long row0,
                            long long group, long long stride, cudaStream_t stream) {
    const int g = grid_for(rows * cols);
    if (dst_type == WT_F32)
        convert_rows_kernel<TS, float><<<g, 256, 0, stream>>>((const TS*)src, (float*)dst, rows, cols, row0, group, stride);
    else if (dst_type == WT_BF16)
        convert_rows_kernel<TS, bf16><<<g, 256, 0, stream>>>((const TS*)src, (bf16*)dst, rows, cols, row0, group, stride);
    else
        return FF_ERR_UNSUPPORTED;
    FF_LAUNCH_CHECK();
    return 0;
}

}  // namespace ff

using namespace ff;

// Map `path` read-only and try to register the mapping with the driver as read-only host memory, as
// the reference does.  register_it == 0 skips the registration (pageable memory; copies from it are
// staged by the driver).  Returns a handle, or null with *err set to errno.  *pinned tells which of
// the two it became (a refused registration leaves its cudaError_t, negated, there: not an error, the
// file stays pageable).  A writable private mapping could be registered where the read-only form is
// refused, but pinning it costs more than it saves (6 s for 16 GB on the machines this was measured
// on, where the pageable copies of the whole file take 1.5 s).
FF_EXPORT void* ff_weights_map_file(const char* path, int register_it, void** addr, unsigned long long* size,
                                    int* pinned, int* err) {
    *err = 0;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) { *err = errno; return nullptr; }
    struct stat st;
    if (fstat(fd, &st) != 0) { *err = errno; close(fd); return nullptr; }
    void* p = st.st_size > 0 ? mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0) : nullptr;
    close(fd);
    if (st.st_size > 0 && p == MAP_FAILED) { *err = errno; return nullptr; }
    MappedFile* m = new MappedFile{p, (size_t)st.st_size, 0};
    int refused = 0;
    if (register_it && p != nullptr) {
        const cudaError_t e = cudaHostRegister(p, m->size, cudaHostRegisterReadOnly | cudaHostRegisterPortable);
        if (e == cudaSuccess) m->pinned = 1;
        else { (void)cudaGetLastError(); refused = -(int)e; }
    }
    *addr = p;
    *size = (unsigned long long)m->size;
    *pinned = m->pinned ? 1 : refused;
    return m;
}

// The caller has waited for every copy that reads the mapping.
FF_EXPORT void ff_weights_unmap_file(void* handle) {
    MappedFile* m = static_cast<MappedFile*>(handle);
    if (m == nullptr) return;
    if (m->pinned) (void)cudaHostUnregister(m->addr);
    if (m->addr != nullptr) munmap(m->addr, m->size);
    delete m;
}

// Copy `rows` rows of `row_bytes` bytes from host memory to their places in a device matrix whose
// rows are `row_bytes` long too (see the row placement above).  One cudaMemcpyAsync for a plain
// block, one cudaMemcpy2DAsync for grouped rows.
FF_EXPORT int ff_weights_copy_rows(void* dst, const void* src, long long rows, long long row_bytes, long long dst_row0,
                                   long long group, long long group_stride, cudaStream_t stream) {
    if (rows <= 0 || row_bytes <= 0) return 0;
    if (group <= 0 || dst_row0 < 0) return FF_ERR_BAD_ARG;
    char* d = static_cast<char*>(dst) + dst_row0 * row_bytes;
    if (group >= rows)
        return (int)cudaMemcpyAsync(d, src, (size_t)(rows * row_bytes), cudaMemcpyHostToDevice, stream);
    if (rows % group != 0 || group_stride < group) return FF_ERR_BAD_ARG;
    return (int)cudaMemcpy2DAsync(d, (size_t)(group_stride * row_bytes), src, (size_t)(group * row_bytes),
                                  (size_t)(group * row_bytes), (size_t)(rows / group), cudaMemcpyHostToDevice, stream);
}

// Convert rows that already lie on the device (a staging buffer, contiguous) into their places.
FF_EXPORT int ff_weights_convert_rows(const void* src, int src_type, void* dst, int dst_type, long long rows,
                                      long long cols, long long dst_row0, long long group, long long group_stride,
                                      cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (group <= 0 || dst_row0 < 0 || (group < rows && group_stride < group)) return FF_ERR_BAD_ARG;
    switch (src_type) {
        case WT_F32: return convert_dispatch<float>(src, dst, dst_type, rows, cols, dst_row0, group, group_stride, stream);
        case WT_BF16: return convert_dispatch<bf16>(src, dst, dst_type, rows, cols, dst_row0, group, group_stride, stream);
        case WT_F16: return convert_dispatch<__half>(src, dst, dst_type, rows, cols, dst_row0, group, group_stride, stream);
        case WT_F64: return convert_dispatch<double>(src, dst, dst_type, rows, cols, dst_row0, group, group_stride, stream);
        default: return FF_ERR_UNSUPPORTED;
    }
}

// Draw a tensor of rows x cols values N(shift, scale) (see above) into its places; via_bf16: rounded to
// bfloat16 on the way, whatever the destination type.
FF_EXPORT int ff_weights_random_rows(void* dst, int dst_type, long long rows, long long cols, long long dst_row0,
                                     long long group, long long group_stride, unsigned long long key,
                                     const int* table, float scale, float shift, int via_bf16, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (group <= 0 || dst_row0 < 0 || table == nullptr) return FF_ERR_BAD_ARG;
    const int g = grid_for(rows * cols);
    if (dst_type == WT_F32)
        random_rows_kernel<float><<<g, 256, 0, stream>>>((float*)dst, rows, cols, dst_row0, group, group_stride, key, table,
                                                         scale, shift, via_bf16);
    else if (dst_type == WT_BF16)
        random_rows_kernel<bf16><<<g, 256, 0, stream>>>((bf16*)dst, rows, cols, dst_row0, group, group_stride, key, table,
                                                        scale, shift, via_bf16);
    else
        return FF_ERR_UNSUPPORTED;
    FF_LAUNCH_CHECK();
    return 0;
}

FF_EXPORT int ff_weights_random_ints(int* dst, long long n, unsigned long long key, unsigned long long high,
                                     cudaStream_t stream) {
    if (n <= 0) return 0;
    if (high == 0) return FF_ERR_BAD_ARG;
    random_int_rows_kernel<<<grid_for(n), 256, 0, stream>>>(dst, n, key, high);
    FF_LAUNCH_CHECK();
    return 0;
}
