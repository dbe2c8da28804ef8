// Plain attention over the paged cache: one block per (query token, q head), scalar
// 32-bit arithmetic throughout.  It serves the true 32-bit path and stands beside
// the tensor-core kernel as its reference.  Any head size up to 256, any block
// size, any group size; prefill portions and decode tokens alike, since every
// query is described only by its sequence and absolute position.
//
// Formula as in the reference's decode kernel (src/kernels/attention.cu:291-447):
// s_j = (q.k_j)/sqrt(d) in 32-bit, running max and sum, o = sum p_j v_j / l, q head
// h reading kv head h / (nq/nkv) (:304).  Unlike the reference's prefill kernel
// (:173, mask on indices local to the portion) keys are taken from the cache by
// absolute position, 0..pos, or the last `window` of them.
//
// A warp takes every 4th key starting at the first visible one, so the order of
// additions for a query depends only on its position and window, never on how the
// tokens were cut into steps or what else is in the batch.
#include "common.cuh"
#include <math_constants.h>

namespace ff {

constexpr int ATT_WARPS = 4;
constexpr int ATT_MAX_D = 256;
constexpr int ATT_PER_LANE = ATT_MAX_D / 32;

template <typename T>
__global__ void paged_attention_simt_kernel(
    const T* __restrict__ q, int q_stride, const T* __restrict__ cache,
    const int* __restrict__ block_table, int max_blocks, const int* __restrict__ token_seq,
    const int* __restrict__ positions, T* __restrict__ out, int out_stride, int nq, int nkv, int d,
    int block_size, int num_blocks, float scale, int window, int* __restrict__ status) {
    pdl_prologue();
    __shared__ float s_m[ATT_WARPS], s_l[ATT_WARPS];
    __shared__ float s_acc[ATT_WARPS][ATT_MAX_D];
    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kh = h / (nq / nkv);
    const int seq = token_seq[t], pos = positions[t];
    const int kv_begin = window > 0 ? max(0, pos - window + 1) : 0;
    const int kv_end = pos + 1;

    float qr[ATT_PER_LANE], acc[ATT_PER_LANE];
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * d;
#pragma unroll
    for (int jj = 0; jj < ATT_PER_LANE; ++jj) {
        const int i = lane + 32 * jj;
        qr[jj] = i < d ? to_float(qrow[i]) : 0.f;
        acc[jj] = 0.f;
    }
    float m = -CUDART_INF_F, l = 0.f;
    const int* bt = block_table + (size_t)seq * max_blocks;
    for (int j = kv_begin + warp; j < kv_end; j += ATT_WARPS) {
        const int page = bt[j / block_size];
        if (page < 0 || page >= num_blocks) {
            if (lane == 0) atomicExch(status, 4);
            break;
        }
        const T* krow = cache + ((((size_t)page * 2) * nkv + kh) * block_size + j % block_size) * d;
        const T* vrow = krow + (size_t)nkv * block_size * d;
        float part = 0.f;
#pragma unroll
        for (int jj = 0; jj < ATT_PER_LANE; ++jj) {
            const int i = lane + 32 * jj;
            if (i < d) part += qr[jj] * to_float(krow[i]);
        }
        const float s = warp_sum(part) * scale;
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);
        const float p = expf(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int jj = 0; jj < ATT_PER_LANE; ++jj) {
            const int i = lane + 32 * jj;
            if (i < d) acc[jj] = acc[jj] * corr + p * to_float(vrow[i]);
        }
        m = m_new;
    }
    if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
    for (int jj = 0; jj < ATT_PER_LANE; ++jj) {
        const int i = lane + 32 * jj;
        if (i < d) s_acc[warp][i] = acc[jj];
    }
    __syncthreads();
    float M = s_m[0];
#pragma unroll
    for (int w = 1; w < ATT_WARPS; ++w) M = fmaxf(M, s_m[w]);
    float wgt[ATT_WARPS], L = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
        wgt[w] = s_m[w] == -CUDART_INF_F ? 0.f : expf(s_m[w] - M);
        L += wgt[w] * s_l[w];
    }
    T* orow = out + (size_t)t * out_stride + (size_t)h * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) o += wgt[w] * s_acc[w][i];
        orow[i] = from_float<T>(o / L);
    }
}

}  // namespace ff

using namespace ff;

FF_EXPORT int ff_paged_attention_simt(const void* q, int dtype, int q_stride, const void* cache,
                                      const int* block_table, int max_blocks, const int* token_seq,
                                      const int* positions, void* out, int out_stride, int T, int nq,
                                      int nkv, int d, int block_size, int num_blocks, float scale,
                                      int window, int* status, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || d > ATT_MAX_D) return FF_ERR_UNSUPPORTED;
    if (nkv <= 0 || nq % nkv) return FF_ERR_BAD_ARG;
    dim3 grid(T, nq);
    if (dtype == 0)
        FF_LAUNCH((paged_attention_simt_kernel<float>), grid, ATT_WARPS * 32, 0, stream, 
            (const float*)q, q_stride, (const float*)cache, block_table, max_blocks, token_seq,
            positions, (float*)out, out_stride, nq, nkv, d, block_size, num_blocks, scale, window, status);
    else if (dtype == 1)
        FF_LAUNCH((paged_attention_simt_kernel<bf16>), grid, ATT_WARPS * 32, 0, stream, 
            (const bf16*)q, q_stride, (const bf16*)cache, block_table, max_blocks, token_seq,
            positions, (bf16*)out, out_stride, nq, nkv, d, block_size, num_blocks, scale, window, status);
    else
        return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}
