// out[t, n] = sum_k x[t, k] * W[n, k] for steps of about a hundred to a few hundred tokens, on
// pairs of SMs: tcgen05.mma with cta_group::2.
//
// Two blocks of a cluster work on one tile of 256 weight rows x NTOK tokens.  Each loads its own
// 128 weight rows (the MMA's M operand) and its own half of the tokens (the N operand) by TMA; the
// instruction, issued by the pair's first block, multiplies both blocks' weight rows with both halves
// of the tokens and leaves each block's 128 x NTOK accumulator in that block's tensor memory.  A
// token tile is thus read from L2 once per 256 weight rows instead of once per 128, which is what
// bounds a one-block tile at these token counts (at 256 tokens a 128-row tile moves three bytes
// through L2 for every weight byte, a pair two).  No load uses cluster multicast: each block fetches
// what it needs itself, the loads' completion is counted on the first block's barrier
// (cp.async.bulk.tensor with cta_group::2), and the MMA's completion is signalled to both blocks
// (tcgen05.commit with a cluster mask).  Matrices with few row tiles are cut into K ranges over more
// blocks of the same cluster (2 x ranges, at most 8), whose partial tiles are summed through
// distributed shared memory in a fixed order, as in the one-block kernel (gemm_tcgen05.cu).
//
// Epilogues and the folded RMSNorm are the one-block kernel's: store bfloat16, store float32, add into
// a float32 residual (optionally leaving bfloat16(residual * w) and per-tile sums of squares for the
// norm that follows), SiLU(gate) * up for a weight whose rows interleave gate and up in groups of 16;
// and on the consuming side the accumulator scaled by 1/rms of the token.
//
// Every wait on an mbarrier is bounded (codes 111 to 113 in the status word); a block that gives up
// still meets its peers at the cluster barriers, lets its copies land and frees its tensor memory.
#include "tcgen05.cuh"

namespace ff {

constexpr int PM = 128;              // weight rows per block; a pair's tile has 2 * PM
constexpr int PAIR_THREADS = 192;
enum PairEpilogue { P_BF16 = 0, P_F32 = 1, P_RESIDUAL_ADD = 2, P_SWIGLU = 3 };

template <int NTOK> struct PairCfg {
    static constexpr int A_BYTES = PM * BK * 2;                 // 16 KB
    static constexpr int B_BYTES = (NTOK / 2) * BK * 2;         // this block's half of the tokens
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    // pipeline depth: nearly all of an SM's shared memory (DEEP: one block per SM, what every launch
    // uses) or half of it (SHALLOW: two blocks per SM, which made a product with between one and two
    // blocks per SM 10 % faster when it ran alone, but two pairs on one pair of SMs both allocate tensor
    // memory across the two SMs, and inside the model's step, where blocks arrive one by one behind the
    // kernel in front, such launches now and then never came back: not used)
    static constexpr int DEEP = (int)((200 * 1024) / STAGE_BYTES) > 8 ? 8 : (int)((200 * 1024) / STAGE_BYTES);
    static constexpr int SHALLOW = (int)((100 * 1024) / STAGE_BYTES);
    static constexpr int TMEM_COLS = NTOK < 32 ? 32 : NTOK;
    // the partial tile of a K range (float [NTOK][PM]) and the epilogue's staging buffer reuse the stages' memory
    static constexpr bool can_split(int stages) { return (size_t)stages * STAGE_BYTES >= (size_t)NTOK * PM * 4 + 32 * PM * 4; }
    static constexpr size_t smem(int stages) { return (size_t)stages * STAGE_BYTES + 1024 + 256; }
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// TMA load whose completion is counted on the barrier at the same place in the pair's first block
// (the barrier's address with the pair bit cleared).
__device__ __forceinline__ void tma_load_2d_pair(bool issue, uint32_t dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t bar_local) {
    const uint32_t bar = bar_local & 0xFEFFFFFFu;
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                 "@q cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n\t}"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"((uint32_t)issue) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(bool issue, uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                                 uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                 "@q tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"((uint32_t)issue) : "memory");
}
// the MMAs issued so far are complete: arrive on the barrier at this place in both blocks of the pair
__device__ __forceinline__ void tc_commit_pair(bool issue, uint32_t bar_local, uint16_t cta_mask) {
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t"
                 "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n\t}"
                 ::"r"(bar_local), "h"(cta_mask), "r"((uint32_t)issue) : "memory");
}
// M = 256 over the pair, N = ntok; bfloat16 operands, float32 accumulator, both K-major
__device__ __forceinline__ uint32_t instr_desc_pair(int ntok) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(ntok >> 3) << 17) | ((uint32_t)((2 * PM) >> 4) << 24);
}

struct PairArgs {
    void* out;
    int ldo;
    int T, N, K;
    int epilogue;
    int ranges;           // K ranges = pairs per cluster (cluster = 2 * ranges blocks)
    int kb_per_range;
    int stages;           // depth of the load pipeline
    int* status;
    bf16* xw_out;         // norm folded in, producing side (see gemm_tcgen05.cu)
    const float* xw_w;
    float* ssq_out;
    const float* ssq_in;  // consuming side
    int ssq_parts;
    int norm_dim;
    float norm_eps;
};

// grid (2 * ranges, row tiles of 256, token tiles); cluster (2 * ranges, 1, 1): block x of a cluster is
// K range x / 2, half x % 2 of its pair.
template <int NTOK>
__global__ void __launch_bounds__(PAIR_THREADS)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const PairArgs a) {
    using Cfg = PairCfg<NTOK>;
    const int STAGES = a.stages;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + (size_t)STAGES * Cfg::STAGE_BYTES);
    // bars[0..S) full (used in the pair's first block), bars[S..2S) empty, bars[2S] accumulator ready
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ float s_inv[NTOK];

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const bool issue = lane == 0;
    const uint32_t crank = cluster_ctarank();
    const int half = (int)(crank & 1u);                  // which block of the pair
    const int range = (int)(crank >> 1);                 // which K range
    const bool leader = half == 0;
    const uint16_t pair_mask = (uint16_t)(3u << (crank & ~1u));
    const int n0 = blockIdx.y * 2 * PM + half * PM;      // this block's weight rows
    const int t0 = blockIdx.z * NTOK;                    // the tile's tokens; this block loads half of them
    const int tb = t0 + half * (NTOK / 2);
    const int num_kb = (a.K + BK - 1) / BK;
    const int kb0 = range * a.kb_per_range;
    const int kb1 = min(num_kb, kb0 + a.kb_per_range);
    const int n_iters = max(0, kb1 - kb0);
    // Every row tile walks its K range from another starting point (and wraps around): all tiles read the
    // same token tile, and in step they would all ask the same few L2 lines of it at the same moment.
    const int rot = n_iters > 0 ? (int)((blockIdx.y * 11u + blockIdx.z * 5u) % (unsigned)n_iters) : 0;
    auto kb_of = [&](int it) { const int k = it + rot; return kb0 + (k >= n_iters ? k - n_iters : k); };

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int i = 0; i < 2 * STAGES + 1; ++i) mbar_init(smem_addr(&bars[i]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // tensor memory of the pair: the same columns in both blocks
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_addr(&s_tmem_base)), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();            // every block's barriers exist before anything arrives on them from outside
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    volatile int* abort_flag = &s_abort;
    grid_launch_dependents();

    float res_pre[16];
    float wn_pre = 0.f;
    if (warp == 0) {
        // ------------------------------------------------ producer: TMA loads --
        int issued = 0;
        const int pre = min(n_iters, STAGES);
        for (int it = 0; it < pre; ++it) {
            const uint32_t full = smem_addr(&bars[it]);
            if (leader) mbar_expect_tx(issue, full, 2 * Cfg::STAGE_BYTES);          // both blocks' bytes
            tma_load_2d_pair(issue, smem_addr(tiles + (size_t)it * Cfg::STAGE_BYTES), &map_w, kb_of(it) * BK, n0, full);
        }
        grid_dependency_wait();
        for (int it = 0; it < pre; ++it) {
            tma_load_2d_pair(issue, smem_addr(tiles + (size_t)it * Cfg::STAGE_BYTES + Cfg::A_BYTES), &map_x, kb_of(it) * BK, tb,
                             smem_addr(&bars[it]));
            issued = it + 1;
        }
        for (int it = pre; it < n_iters; ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            if (!__all_sync(0xffffffffu, mbar_wait(smem_addr(&bars[STAGES + s]), ph ^ 1, a.status, abort_flag, 111))) break;
            const uint32_t full = smem_addr(&bars[s]);
            if (leader) mbar_expect_tx(issue, full, 2 * Cfg::STAGE_BYTES);
            unsigned char* st = tiles + (size_t)s * Cfg::STAGE_BYTES;
            tma_load_2d_pair(issue, smem_addr(st), &map_w, kb_of(it) * BK, n0, full);
            tma_load_2d_pair(issue, smem_addr(st + Cfg::A_BYTES), &map_x, kb_of(it) * BK, tb, full);
            issued = it + 1;
        }
        (void)issued;
    } else if (warp == 1 && leader) {
        // ------------------------------------------------ MMA issuer (first block of the pair) --
        const uint32_t idesc = instr_desc_pair(NTOK);
        bool ok = true;
        for (int it = 0; it < n_iters && ok; ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            ok = __all_sync(0xffffffffu, mbar_wait(smem_addr(&bars[s]), ph, a.status, abort_flag, 112));
            if (!ok) break;
            tc_fence_after();
            const uint32_t sa = smem_addr(tiles + (size_t)s * Cfg::STAGE_BYTES);
            const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
                const uint64_t da = smem_desc_sw128(sa + k * UMMA_K * 2);
                const uint64_t db = smem_desc_sw128(sb + k * UMMA_K * 2);
                tc_mma_bf16_pair(issue, tmem_base, da, db, idesc, (it > 0 || k > 0) ? 1u : 0u);
            }
            tc_commit_pair(issue, smem_addr(&bars[STAGES + s]), pair_mask);     // the stage is free in both blocks
            __syncwarp();
        }
        tc_commit_pair(issue, smem_addr(&bars[2 * STAGES]), pair_mask);         // both accumulators are complete
    } else if (warp >= 2) {
        // ------------------------------------------------ epilogue warps, while the main loop runs --
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int n = n0 + row;
        bool ok = true;
        if (a.ssq_in) {
            grid_dependency_wait();
            const int et = threadIdx.x - 64;
            for (int c = et; c < NTOK; c += 128) {
                const int t = t0 + c;
                float ss = 0.f;
                if (t < a.T) {
#pragma unroll 8
                    for (int p = 0; p < a.ssq_parts; ++p) ss += __ldcg(a.ssq_in + (size_t)p * a.T + t);
                }
                s_inv[c] = 1.0f / sqrtf(ss / (float)a.norm_dim + a.norm_eps);
            }
        }
        if (a.epilogue == P_RESIDUAL_ADD) {
            grid_dependency_wait();
            int c_begin = 0, c_end = NTOK;
            if (a.ranges > 1) {
                const int per = (NTOK + a.ranges - 1) / a.ranges;
                c_begin = min(NTOK, range * per);
                c_end = min(NTOK, c_begin + per);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int t = t0 + c_begin + i;
                res_pre[i] = (c_begin + i < c_end && t < a.T && n < a.N)
                                 ? __ldcg(reinterpret_cast<const float*>(a.out) + (size_t)t * a.ldo + n) : 0.f;
            }
            if (a.xw_out && n < a.N) wn_pre = __ldg(a.xw_w + n);
        }
        if (n_iters > 0) ok = mbar_wait(smem_addr(&bars[2 * STAGES]), 0, a.status, abort_flag, 113);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        if (a.ranges > 1) {
            // this block's partial tile -> its own shared memory (the stages are free now), [token][row]
            float* mine = reinterpret_cast<float*>(tiles);
#pragma unroll 1
            for (int c0 = 0; c0 < NTOK; c0 += 16) {
                float v[16];
                if (n_iters > 0 && ok) tc_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + c0, v);
                else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = 0.f;
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) mine[(c0 + i) * PM + row] = v[i];
            }
        }
    }
    if (a.ranges > 1) cluster_sync_all();          // every block's partial tile is in place
    if (warp >= 2) {
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int n = n0 + row;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool ok = !*abort_flag;
        grid_dependency_wait();
        int c_begin = 0, c_end = NTOK;
        if (a.ranges > 1) {
            const int per = (NTOK + a.ranges - 1) / a.ranges;
            c_begin = min(NTOK, range * per);
            c_end = min(NTOK, c_begin + per);
        }
        const uint32_t mine_addr = smem_addr(tiles);
        // The accumulator has a weight row per thread and a token per register, the output a token per row
        // of memory: written from the registers, a warp's store would be 32 two-byte pieces 64 bytes apart
        // in time (at 256 tokens that alone took as long as the whole main loop).  So the tile passes
        // through shared memory 32 tokens at a time, float [32][SROW], and leaves it with a thread writing
        // 32 consecutive rows of one token: whole 16-byte vectors, four threads to a token's 128 rows.
        constexpr int CH = 32, SROW = PM;                  // rows swizzled by the token: see below
        float* stage = reinterpret_cast<float*>(tiles + (a.ranges > 1 ? (size_t)NTOK * PM * 4 : 0));
        const int et = threadIdx.x - 64;                   // 0..127
        const int o_tok = et >> 2, o_rg = et & 3;          // this thread's token of the chunk and group of 32 rows on the way out
        const int o_n = n0 + o_rg * 32;
        (void)res_pre; (void)wn_pre; (void)n;
#pragma unroll 1
        for (int c0 = c_begin; c0 < c_end; c0 += CH) {
            // ---- in: this thread's row, 32 tokens ----
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int cc = c0 + h * 16;
                float v[16];
                const int cn = max(0, min(16, c_end - cc));
                if (a.ranges == 1) {
                    if (n_iters > 0 && ok && cn > 0) tc_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + cc, v);
                    else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = 0.f;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = 0.f;
                    // the same half of every pair of the cluster, in the order of the K ranges
                    for (int z = 0; z < a.ranges; z += 2) {
                        float p0[16], p1[16];
                        const bool two = z + 1 < a.ranges;
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const uint32_t addr = mine_addr + (uint32_t)((cc + i) * PM + row) * 4u;
                            p0[i] = i < cn ? ld_peer_smem(addr, (uint32_t)(2 * z + half)) : 0.f;
                            p1[i] = (two && i < cn) ? ld_peer_smem(addr, (uint32_t)(2 * (z + 1) + half)) : 0.f;
                        }
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            v[i] += p0[i];
                            if (two) v[i] += p1[i];
                        }
                    }
                }
                if (a.ssq_in) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] *= s_inv[min(cc + i, NTOK - 1)];
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) stage[(h * 16 + i) * SROW + (row ^ (((h * 16 + i) & 7) << 2))] = v[i];
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            // ---- out: one token, 32 consecutive rows ----
            const int c = c0 + o_tok, t = t0 + c;
            if (ok && c < c_end && t < a.T) {
                float r[32];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    // groups of four rows sit at (group ^ token % 8): a warp's 32 reads of 16 bytes then spread
                    // evenly over the banks, and so did the writes above
                    const float4 q = *reinterpret_cast<const float4*>(stage + o_tok * SROW + ((o_rg * 32 + j * 4) ^ ((o_tok & 7) << 2)));
                    r[j * 4] = q.x; r[j * 4 + 1] = q.y; r[j * 4 + 2] = q.z; r[j * 4 + 3] = q.w;
                }
#ifdef FF_PAIR_NO_STORE
                if (r[0] == 123.456f)
#endif
                if (a.epilogue == P_SWIGLU) {
                    // the 32 rows are 16 gate rows and the 16 up rows of the same columns
                    const int col = o_n / 2;
                    if (col < a.N / 2) {
                        uint32_t w[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float g0 = r[2 * i], g1 = r[2 * i + 1];
                            __nv_bfloat162 pk = __floats2bfloat162_rn(g0 / (1.0f + expf(-g0)) * r[16 + 2 * i],
                                                                      g1 / (1.0f + expf(-g1)) * r[17 + 2 * i]);
                            w[i] = *reinterpret_cast<uint32_t*>(&pk);
                        }
                        bf16* dst = reinterpret_cast<bf16*>(a.out) + (size_t)t * a.ldo + col;
                        if (col + 16 <= a.N / 2 && (((uintptr_t)dst) & 15) == 0) {
                            reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                            reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (col + i < a.N / 2) dst[i] = __ushort_as_bfloat16((unsigned short)(w[i >> 1] >> ((i & 1) * 16)));
                        }
                    }
                } else if (a.epilogue == P_BF16) {
                    bf16* dst = reinterpret_cast<bf16*>(a.out) + (size_t)t * a.ldo + o_n;
                    if (o_n + 32 <= a.N && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t w[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                __nv_bfloat162 pk = __floats2bfloat162_rn(r[j * 8 + 2 * i], r[j * 8 + 2 * i + 1]);
                                w[i] = *reinterpret_cast<uint32_t*>(&pk);
                            }
                            reinterpret_cast<uint4*>(dst)[j] = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (o_n + i < a.N) dst[i] = __float2bfloat16_rn(r[i]);
                    }
                } else {
                    // float32 out: store, or add into the residual (and prepare the norm that follows)
                    float* dst = reinterpret_cast<float*>(a.out) + (size_t)t * a.ldo + o_n;
                    const bool whole = o_n + 32 <= a.N && (((uintptr_t)dst) & 15) == 0;
                    float sq = 0.f;
                    if (a.epilogue == P_RESIDUAL_ADD) {
                        if (whole) {
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const float4 q = __ldcg(reinterpret_cast<const float4*>(dst) + j);
                                r[j * 4] += q.x; r[j * 4 + 1] += q.y; r[j * 4 + 2] += q.z; r[j * 4 + 3] += q.w;
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (o_n + i < a.N) r[i] += dst[i];
                        }
                    }
                    if (whole) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            reinterpret_cast<float4*>(dst)[j] = make_float4(r[j * 4], r[j * 4 + 1], r[j * 4 + 2], r[j * 4 + 3]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (o_n + i < a.N) dst[i] = r[i];
                    }
                    if (a.xw_out) {
                        bf16* xd = a.xw_out + (size_t)t * a.N + o_n;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            if (o_n + i < a.N) {
                                xd[i] = __float2bfloat16_rn(r[i] * __ldg(a.xw_w + o_n + i));
                                sq += r[i] * r[i];
                            }
                        }
                    }
                    if (a.xw_out) {
                        // the four threads of a token hold its 128 rows: one row of sums per 128 weight rows
                        sq += __shfl_xor_sync(0xffffffffu, sq, 1);
                        sq += __shfl_xor_sync(0xffffffffu, sq, 2);
                        if (o_rg == 0) a.ssq_out[(size_t)(n0 / PM) * a.T + t] = sq;
                    }
                }
            } else if (a.xw_out && a.epilogue == P_RESIDUAL_ADD) {
                float sq = 0.f;                            // keep the shuffles of the branch above warp-wide
                sq += __shfl_xor_sync(0xffffffffu, sq, 1);
                sq += __shfl_xor_sync(0xffffffffu, sq, 2);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
    }
    // peers may still be reading this block's partial tile, and the pair's tensor memory is freed together
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
    }
}

template <int NTOK>
static int launch_pair(const CUtensorMap& mw, const CUtensorMap& mx, const PairArgs& a_in, int row_tiles, int t_tiles, int pdl,
                       cudaStream_t stream) {
    using Cfg = PairCfg<NTOK>;
    PairArgs a = a_in;
    // one wave of blocks at one per SM -> deep pipelines; more blocks than SMs (and no K ranges, whose
    // partial tiles need the room) -> two per SM
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long blocks = 2ll * a.ranges * row_tiles * t_tiles;
    (void)blocks;
    a.stages = Cfg::DEEP;
    if (a.stages < 2) a.stages = 2;
    if (a.ranges > 1 && !Cfg::can_split(a.stages)) return FF_ERR_UNSUPPORTED;
    FF_SMEM_LIMIT(gemm_pair_kernel<NTOK>, Cfg::smem(Cfg::DEEP));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * a.ranges, row_tiles, t_tiles);
    cfg.blockDim = dim3(PAIR_THREADS);
    cfg.dynamicSmemBytes = Cfg::smem(a.stages);
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    int na = 0;
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = 2 * a.ranges;
    attrs[na].val.clusterDim.y = 1;
    attrs[na].val.clusterDim.z = 1;
    ++na;
    if (pdl || g_ff_pdl) {
        attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel<NTOK>, mw, mx, a);
    if (e != cudaSuccess) return (int)e;
    return 0;
}

}  // namespace ff

using namespace ff;

// Tokens per tile (64, 128 or 256) and K ranges (1 to 4) a call would use.
FF_EXPORT int ff_gemm_pair_plan(int T, int N, int K, int want_ranges, int* ntok_out, int* ranges_out) {
    int ntok = 64;
    while (ntok < T && ntok < 256) ntok <<= 1;
    const int num_kb = (K + BK - 1) / BK;
    int ranges = want_ranges < 1 ? 1 : (want_ranges > 4 ? 4 : want_ranges);
    if (ranges > num_kb) ranges = num_kb;
    const int per = (num_kb + ranges - 1) / ranges;
    ranges = (num_kb + per - 1) / per;
    *ntok_out = ntok;
    *ranges_out = ranges;
    return 0;
}

// Arguments as ff_gemm_tc (gemm_tcgen05.cu); `want_ranges` K ranges (at most 4: the cluster holds two
// blocks per range).
FF_EXPORT int ff_gemm_pair(const void* x, const void* w, void* out, int ldo, int T, int N, int K, int epilogue,
                           int want_ranges, int pdl, void* xw_out, const float* xw_w, float* ssq_out,
                           const float* ssq_in, int ssq_parts, int norm_dim, float norm_eps, int* status,
                           cudaStream_t stream) {
    if (xw_out && (epilogue != P_RESIDUAL_ADD || !xw_w || !ssq_out)) return FF_ERR_BAD_ARG;
    if (ssq_in && (ssq_parts <= 0 || norm_dim <= 0)) return FF_ERR_BAD_ARG;
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0 || (K % 8) || epilogue < 0 || epilogue > 3) return FF_ERR_BAD_ARG;
    if (epilogue == P_SWIGLU && (N % 32)) return FF_ERR_UNSUPPORTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return FF_ERR_BAD_ARG;
    int ntok, ranges;
    ff_gemm_pair_plan(T, N, K, want_ranges, &ntok, &ranges);
    const int row_tiles = (N + 2 * PM - 1) / (2 * PM), t_tiles = (T + ntok - 1) / ntok;
    const int num_kb = (K + BK - 1) / BK;
    CUtensorMap mw, mx;
    int rc = make_map(w, N, K, PM, &mw);
    if (rc) return rc;
    rc = make_map(x, T, K, ntok / 2, &mx);
    if (rc) return rc;
    PairArgs a;
    a.out = out; a.ldo = ldo; a.T = T; a.N = N; a.K = K; a.epilogue = epilogue; a.ranges = ranges;
    a.kb_per_range = (num_kb + ranges - 1) / ranges;
    a.status = status;
    a.xw_out = (bf16*)xw_out; a.xw_w = xw_w; a.ssq_out = ssq_out;
    a.ssq_in = ssq_in; a.ssq_parts = ssq_parts; a.norm_dim = norm_dim; a.norm_eps = norm_eps;
    switch (ntok) {
        case 64: return launch_pair<64>(mw, mx, a, row_tiles, t_tiles, pdl, stream);
        case 128: return launch_pair<128>(mw, mx, a, row_tiles, t_tiles, pdl, stream);
        default: return launch_pair<256>(mw, mx, a, row_tiles, t_tiles, pdl, stream);
    }
}
