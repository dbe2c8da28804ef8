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

constexpr int SAMPLE_THREADS = 256;

__device__ __forceinline__ float gumbel_noise(uint64_t seed, uint64_t counter, uint32_t i) {
    const uint64_t r = mix64(mix64(seed) ^ mix64(counter * 0x100000001B3ull + i));
    const float u = ((float)(uint32_t)(r >> 40) + 0.5f) * (1.0f / 16777216.0f);  // (0,1), 24 bits
    return -logf(-logf(u));
}

// (best value, its index) over elements [lo, hi) of a row; ties go to the lowest index
__device__ __forceinline__ void scan_range(const float* __restrict__ row, int lo, int hi, bool greedy, float inv_t,
                                           uint64_t seed, uint64_t ctr, float& best, int& best_i) {
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        float x = row[i];
        if (!greedy) x = x * inv_t + gumbel_noise(seed, ctr, (uint32_t)i);
        if (x > best) { best = x; best_i = i; }  // strict: the lowest index of a thread's ties stays
    }
}

__device__ __forceinline__ void better(float& best, int& best_i, float ov, int oi) {
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
}

// Reduce (best, best_i) over the block; the result is valid in thread 0.
__device__ __forceinline__ void block_best(float& best, int& best_i, float* s_val, int* s_idx) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        better(best, best_i, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, best_i, o));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        best = lane < nw ? s_val[lane] : -CUDART_INF_F;
        best_i = lane < nw ? s_idx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            better(best, best_i, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, best_i, o));
    }
}

// grid (rows, chunks).  With one chunk the token is written at once; else each block leaves
// its chunk's best in scratch memory for sample_final_kernel.
__global__ void sample_kernel(const float* __restrict__ logits, int V, size_t row_stride,
                              const float* __restrict__ temperature, const long long* __restrict__ seeds,
                              const long long* __restrict__ counters, int* __restrict__ out,
                              float* __restrict__ part_val, int* __restrict__ part_idx) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    pdl_prologue();      // the logits come from the kernel in front
    const int r = blockIdx.x, chunks = gridDim.y, c = blockIdx.y;
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temperature ? temperature[r] : 0.f;
    const bool greedy = !(temp > 0.f);
    const float inv_t = greedy ? 1.f : 1.f / temp;
    const uint64_t seed = seeds ? (uint64_t)seeds[r] : 0ull;
    const uint64_t ctr = counters ? (uint64_t)counters[r] : 0ull;
    const int per = (V + chunks - 1) / chunks;
    float best = -CUDART_INF_F;
    int best_i = 0x7fffffff;
    scan_range(row, c * per, min(V, (c + 1) * per), greedy, inv_t, seed, ctr, best, best_i);
    block_best(best, best_i, s_val, s_idx);
    if (threadIdx.x == 0) {
        if (chunks == 1) out[r] = best_i == 0x7fffffff ? 0 : best_i;
        else { part_val[r * chunks + c] = best; part_idx[r * chunks + c] = best_i; }
    }
}

__global__ void sample_final_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx,
                                    int chunks, int* __restrict__ out) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    pdl_prologue();      // the chunks' results come from sample_kernel
    const int r = blockIdx.x;
    float best = -CUDART_INF_F;
    int best_i = 0x7fffffff;
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) better(best, best_i, part_val[r * chunks + c], part_idx[r * chunks + c]);
    block_best(best, best_i, s_val, s_idx);
    if (threadIdx.x == 0) out[r] = best_i == 0x7fffffff ? 0 : best_i;
}

}  // namespace ff

using namespace ff;

// temperature / seeds / counters may be null: plain arg-max.  chunks > 1 splits every row over
// that many blocks and needs scratch memory of rows*chunks floats and ints.
FF_EXPORT int ff_sample(const float* logits, int rows, int V, size_t row_stride,
                        const float* temperature, const long long* seeds, const long long* counters,
                        int* out, int chunks, float* part_val, int* part_idx, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (V <= 0 || chunks < 1 || chunks > 1024) return FF_ERR_BAD_ARG;
    if (chunks > 1 && (!part_val || !part_idx)) return FF_ERR_BAD_ARG;
    FF_LAUNCH((sample_kernel), dim3(rows, chunks), SAMPLE_THREADS, 0, stream, logits, V, row_stride, temperature,
              seeds, counters, out, part_val, part_idx);
    if (chunks > 1)
        FF_LAUNCH((sample_final_kernel), rows, 32, 0, stream, (const float*)part_val, (const int*)part_idx, chunks, out);
    return 0;
}
