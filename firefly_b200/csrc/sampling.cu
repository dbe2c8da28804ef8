// Choosing the next token from 32-bit logits: arg-max, and temperature sampling by
// the Gumbel-max rule with counter-based random numbers.
//
// The reference samples greedily only: arg-max with a strict '>' per thread and a
// CUB block reduction (src/kernels/sampling.cu:12-44).  Here ties go to the lowest
// index at every level.  For temperature T > 0 the token is
// argmax_i( logit_i / T + g_i ),  g_i = -log(-log(u_i)),  which draws from
// softmax(logits / T) in one pass with no normalisation; u_i is a hash of
// (seed, counter, i), so a request's draws can be replayed and do not depend on
// the batch it sits in.
#include "common.cuh"
#include <math_constants.h>

namespace ff {

constexpr int SAMPLE_THREADS = 512;

__device__ __forceinline__ float gumbel_noise(uint64_t seed, uint64_t counter, uint32_t i) {
    const uint64_t r = mix64(mix64(seed) ^ mix64(counter * 0x100000001B3ull + i));
    const float u = ((float)(uint32_t)(r >> 40) + 0.5f) * (1.0f / 16777216.0f);  // (0,1), 24 bits
    return -logf(-logf(u));
}

__global__ void sample_kernel(const float* __restrict__ logits, int V, size_t row_stride,
                              const float* __restrict__ temperature, const long long* __restrict__ seeds,
                              const long long* __restrict__ counters, int* __restrict__ out) {
    __shared__ float s_val[SAMPLE_THREADS / 32];
    __shared__ int s_idx[SAMPLE_THREADS / 32];
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temperature ? temperature[r] : 0.f;
    const bool greedy = !(temp > 0.f);
    const float inv_t = greedy ? 1.f : 1.f / temp;
    const uint64_t seed = seeds ? (uint64_t)seeds[r] : 0ull;
    const uint64_t ctr = counters ? (uint64_t)counters[r] : 0ull;
    float best = -CUDART_INF_F;
    int best_i = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        float x = row[i];
        if (!greedy) x = x * inv_t + gumbel_noise(seed, ctr, (uint32_t)i);
        if (x > best) { best = x; best_i = i; }  // strict: the lowest index of a thread's ties stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? s_val[lane] : -CUDART_INF_F;
        best_i = lane < nw ? s_idx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        if (lane == 0) out[r] = best_i == 0x7fffffff ? 0 : best_i;
    }
}

}  // namespace ff

using namespace ff;

// temperature / seeds / counters may be null: plain arg-max.
FF_EXPORT int ff_sample(const float* logits, int rows, int V, size_t row_stride,
                        const float* temperature, const long long* seeds, const long long* counters,
                        int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (V <= 0) return FF_ERR_BAD_ARG;
    sample_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, V, row_stride, temperature, seeds, counters, out);
    FF_LAUNCH_CHECK();
    return 0;
}
