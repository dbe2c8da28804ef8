// ff_attn_decode_static: the split-KV decode attention of attention_mma.cu with its
// scratch memory in a file-scope device array, for callers that cannot allocate
// (see attention_decode_static.h).  The kernels are the same ones; only where the
// partial results live differs.
#include "attention_mma.cu"
#include "attention_decode_static.h"

#include <atomic>
#include <cstdio>
#include <mutex>

namespace {

// per-split partial outputs [partials][D] followed by (max, sum) pairs [partials][2]
__device__ __align__(256) float g_static_part_o[(size_t)FF_ATTN_STATIC_MAX_PARTIALS * ff::D];
__device__ __align__(256) float g_static_part_ml[(size_t)FF_ATTN_STATIC_MAX_PARTIALS * 2];

constexpr int kStaticMaxDevices = 64;
std::mutex g_setup_mutex;
std::atomic<bool> g_ready[kStaticMaxDevices];   // set (release) after the addresses below are written
float* g_part_o_addr[kStaticMaxDevices];
float* g_part_ml_addr[kStaticMaxDevices];

// Once per device, with that device current: the arrays' device addresses (in host
// code the symbols are only stand-ins, never to be handed to a kernel) and the
// kernels' dynamic shared-memory limit.
int setup_device(int dev) {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_ready[dev].load(std::memory_order_acquire)) return 0;
    float* po = nullptr;
    float* pml = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&po, g_static_part_o);
    if (e != cudaSuccess) return (int)e;
    e = cudaGetSymbolAddress((void**)&pml, g_static_part_ml);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(ff::attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)ff::DECODE_SMEM);
    if (e != cudaSuccess) return (int)e;
    g_part_o_addr[dev] = po;
    g_part_ml_addr[dev] = pml;
    g_ready[dev].store(true, std::memory_order_release);
    return 0;
}

}  // namespace

extern "C" __attribute__((visibility("default")))
int ff_attn_decode_static(const void* q, int q_stride, const void* cache, const int* block_table,
                          int max_blocks, const int* cu_q, const int* ctx_lens, int n_seqs, void* out,
                          int out_stride, int nq, int nkv, int block_size, int num_blocks, float scale,
                          int window, int num_splits, cudaStream_t stream) {
    using namespace ff;
    if (n_seqs <= 0) return 0;
    if (nkv <= 0 || nq % nkv || num_splits < 1) return FF_ERR_BAD_ARG;
    if (nq / nkv > 16) return FF_ERR_UNSUPPORTED;
    const long long partials = (long long)n_seqs * nq * num_splits;
    if (partials > FF_ATTN_STATIC_MAX_PARTIALS) {
        std::fprintf(stderr,
                     "ff_attn_decode_static: %d sequences x %d heads x %d splits = %lld partial results "
                     "exceed the built-in scratch array of %d; use fewer splits or ff_attn_decode with "
                     "caller-provided scratch memory\n",
                     n_seqs, nq, num_splits, partials, FF_ATTN_STATIC_MAX_PARTIALS);
        return FF_ATTN_STATIC_TOO_LARGE;
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kStaticMaxDevices) return FF_ERR_UNSUPPORTED;
    if (!g_ready[dev].load(std::memory_order_acquire)) {
        const int rc = setup_device(dev);
        if (rc != 0) return rc;
    }
    float* part_o = g_part_o_addr[dev];
    float* part_ml = g_part_ml_addr[dev];
    dim3 grid(n_seqs, nkv, num_splits);
    attn_decode_kernel<<<grid, NTHREADS, DECODE_SMEM, stream>>>(
        (const bf16*)q, q_stride, (const bf16*)cache, block_table, max_blocks, cu_q, ctx_lens, (bf16*)out,
        out_stride, part_o, part_ml, nq, nkv, block_size, num_blocks, scale * LOG2E, window, num_splits,
        (int*)nullptr);
    FF_LAUNCH_CHECK();
    if (num_splits > 1) {
        dim3 cgrid(n_seqs, nq);
        attn_combine_kernel<<<cgrid, D >= 128 ? 128 : 64, 0, stream>>>(part_o, part_ml, cu_q, (bf16*)out,
                                                                     out_stride, nq, num_splits);
        FF_LAUNCH_CHECK();
    }
    return 0;
}
