// Shared helpers of the sm_100a kernels: element types, reductions, launch checks.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define FF_EXPORT extern "C" __attribute__((visibility("default")))

// error codes returned by the C entry points (0 = ok, >0 = cudaError_t, <0 = ours)
#define FF_ERR_BAD_ARG (-1)
#define FF_ERR_UNSUPPORTED (-2)

#define FF_LAUNCH_CHECK()                         \
    do {                                          \
        cudaError_t _e = cudaGetLastError();      \
        if (_e != cudaSuccess) return (int)_e;    \
    } while (0)

// Programmatic dependent launch.  When switched on (ff_set_pdl(1), per library) every kernel
// is launched with the programmatic-stream-serialization attribute: it may begin while the
// kernel before it in the stream is still running.  Each kernel therefore first lets its own
// dependents start (griddepcontrol.launch_dependents) and then waits for its predecessors to
// finish and their writes to be visible (griddepcontrol.wait) before it touches any memory
// they produce.  In a launch without the attribute both instructions do nothing.
static int g_ff_pdl = 0;
FF_EXPORT void ff_set_pdl(int on) { g_ff_pdl = on; }

namespace ff {

// cluster_z > 1: blocks (x, y, z0..z0+cluster_z) form one thread-block cluster.
template <typename... KArgs, typename... Args>
static inline int launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                        cudaStream_t stream, int cluster_z, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (g_ff_pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (cluster_z > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = (unsigned)cluster_z;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
static inline int launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                cudaStream_t stream, Args... args) {
    return launch_kernel_cluster(kernel, grid, block, smem, stream, 1, args...);
}

// Raise a kernel's dynamic shared-memory limit once per device (a process may use several).
// `flags` is a static array of kMaxDevices bools owned by the call site.
constexpr int kMaxDevices = 64;
template <typename K>
static inline int set_smem_limit_once(K* kernel, size_t bytes, bool* flags) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return FF_ERR_UNSUPPORTED;
    if (flags[dev]) return 0;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
    flags[dev] = true;
    return 0;
}
#define FF_SMEM_LIMIT(kernel, bytes)                                                \
    do {                                                                            \
        static bool _set[ff::kMaxDevices];                                          \
        int _rc = ff::set_smem_limit_once(kernel, (size_t)(bytes), _set);           \
        if (_rc) return _rc;                                                        \
    } while (0)

#define FF_LAUNCH(kernel, grid, block, smem, stream, ...)                                              \
    do {                                                                                               \
        int _rc = ff::launch_kernel(kernel, dim3(grid), dim3(block), (size_t)(smem), stream, __VA_ARGS__); \
        if (_rc) return _rc;                                                                           \
    } while (0)

__device__ __forceinline__ void pdl_prologue() {
    asm volatile("griddepcontrol.launch_dependents;\n\tgriddepcontrol.wait;" ::: "memory");
}

// Barrier over all threads of all blocks of the cluster (release/acquire).
__device__ __forceinline__ void cluster_sync_all() {
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// float at shared-memory address `addr` (as seen by this block) in the block of rank `rank` of the cluster
__device__ __forceinline__ float ld_peer_smem(uint32_t addr, uint32_t rank) {
    uint32_t peer;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(peer) : "memory");
    return v;
}

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(bf16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` is 32 floats of shared memory.  The order of additions is fixed.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : 0.f;
    t = warp_sum(t);
    return t;
}

// 64-bit mix used by the samplers' counter-based random numbers (splitmix64 finaliser).
__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

}  // namespace ff
