// out[t, n] = sum_k x[t, k] * W[n, k]   (y = x W^T, W as stored in checkpoints)
// on the fifth-generation tensor cores: tcgen05.mma with the accumulator in tensor
// memory, operands brought into shared memory by TMA, one lane of a converged warp
// issuing the MMAs, and an epilogue that reads the accumulator back with tcgen05.ld.
//
// The weight tile is the 128-row "M" operand of the MMA and the tokens are its "N"
// dimension (16 to 256), so a decode step with a handful of tokens still fills the
// tensor-core shape and the kernel's time is the time to stream the weights.  For
// matrices with few row tiles the K range is split over the blocks of a thread-block
// cluster (up to 8): each keeps its partial tile in its own shared memory, and after
// a cluster barrier every block adds the partials of a slice of the tokens, in a
// fixed order, reading its peers' shared memory, and runs the epilogue on that
// slice.  No global scratch memory is involved.  Epilogues: store bfloat16, store
// float32, add into a float32 residual, or SiLU(gate)*up for a weight whose rows
// interleave gate and up in groups of 16.  Two optional extras fold an RMSNorm between
// two products into them: the residual-adding product also writes bfloat16(residual*w)
// for the norm that follows and each row tile's sum of squares per token; the product
// that consumes those activations multiplies its accumulator by 1/rms of the token,
// summed from those partial sums in tile order.
//
// The reference runs these products through a library template with half-precision
// accumulation (src/kernels/linear.cu:15-104), followed by separate launches for the
// activation (src/kernels/activation.cu) and the residual add (src/kernels/add.cu).
//
// Every wait on an mbarrier is bounded: after about a second the kernel records an
// error code, stops issuing work, lets its copies land, frees its tensor memory
// and returns.
#include "tcgen05.cuh"

namespace ff {

constexpr int BN = 128;          // weight rows per tile (MMA M)
constexpr int GEMM_THREADS = 192;
// Test builds only (-DFF_GEMM_TEST_DROP_KBLOCK=i): the loads of a block's i-th k block are never
// issued, so the wait for that stage runs out; the test checks that the kernel gives up cleanly.
#ifdef FF_GEMM_TEST_DROP_KBLOCK
#define FF_GEMM_LOADS(it) ((it) != FF_GEMM_TEST_DROP_KBLOCK)
#else
#define FF_GEMM_LOADS(it) true
#endif

enum Epilogue { EPI_BF16 = 0, EPI_F32 = 1, EPI_RESIDUAL_ADD = 2, EPI_SWIGLU = 3 };

constexpr int MAX_STAGES = 12;
constexpr size_t SMEM_BUDGET = 220 * 1024;   // of the 227 KB a block may have

template <int TOK> struct TileCfg {
    static constexpr int A_BYTES = BN * BK * 2;
    static constexpr int B_BYTES = TOK * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TMEM_COLS = TOK < 32 ? 32 : TOK;
    // pipeline depth: half of an SM's shared memory (SHALLOW, what every launch uses: two blocks, of
    // this product or of this and the next one, share an SM) or all of it (DEEP, measured slower)
    static constexpr int DEEP = (SMEM_BUDGET / STAGE_BYTES) > MAX_STAGES ? MAX_STAGES : (int)(SMEM_BUDGET / STAGE_BYTES);
    static constexpr int SHALLOW = (SMEM_BUDGET / 2 / STAGE_BYTES) < 2 ? 2 : (int)(SMEM_BUDGET / 2 / STAGE_BYTES);
    static constexpr size_t smem(int stages) {
        return (size_t)stages * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
    }
};

// Instruction descriptor: bfloat16 x bfloat16 -> float32, both operands K-major, M = 128, N = TOK
__device__ __forceinline__ uint32_t instr_desc(int tok) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(tok >> 3) << 17) | ((uint32_t)(BN >> 4) << 24);
}

struct GemmArgs {
    void* out;
    int ldo;              // elements between rows (tokens) of out
    int T, N, K;
    int epilogue;
    int splits;           // number of K ranges = blocks per cluster (grid.z)
    int kb_per_split;     // 64-wide k blocks per range
    int stages;           // depth of the load pipeline
    int* status;
    // RMSNorm folded in, producing side (EPI_RESIDUAL_ADD only; null: off): after out += acc,
    // xw_out[t, n] = bfloat16(out[t, n] * xw_w[n]) and ssq_out[row tile][t] = sum over the tile's columns of out^2
    bf16* xw_out;
    const float* xw_w;
    float* ssq_out;
    // RMSNorm folded in, consuming side (null: off): the accumulator of token t is multiplied by
    // rsqrt(sum_p ssq_in[p][t] / norm_dim + norm_eps), p < ssq_parts
    const float* ssq_in;
    int ssq_parts;
    int norm_dim;
    float norm_eps;
};

template <int TOK>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               const GemmArgs a) {
    using Cfg = TileCfg<TOK>;
    const int STAGES = a.stages;
    extern __shared__ unsigned char smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + (size_t)STAGES * Cfg::STAGE_BYTES);
    // bars[0..S) full, bars[S..2S) empty, bars[2S] accumulator ready
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ float s_inv[256];          // 1/rms per token of the tile (norm folded in, consuming side)
    __shared__ float s_red[4][16];        // per-warp sums of squares (producing side)

    // the warp index through a shuffle: the compiler then knows it to be the same in the whole warp
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const bool issue = lane == 0;
    const int n0 = blockIdx.x * BN, t0 = blockIdx.y * TOK;
    const int num_kb = (a.K + BK - 1) / BK;
    const int kb0 = blockIdx.z * a.kb_per_split;
    const int kb1 = min(num_kb, kb0 + a.kb_per_split);
    const int n_iters = max(0, kb1 - kb0);

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int i = 0; i < 2 * STAGES + 1; ++i) mbar_init(smem_addr(&bars[i]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // tensor memory for the accumulator: TOK columns of 128 lanes
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_addr(&s_tmem_base)), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    volatile int* abort_flag = &s_abort;
    grid_launch_dependents();

    // what the epilogue adds to (the residual's values of this block's first 16 tokens) and the norm
    // weight of its row, fetched by the epilogue warps while the main loop runs
    float res_pre[16];
    float wn_pre = 0.f;
    if (warp == 0) {
        // ------------------------------------------------ producer: TMA loads --
        // The weights do not depend on the kernel before this one: the first stages' weight
        // tiles are requested at once; the activations only after that kernel has finished.
        int issued = 0;
        const int pre = min(n_iters, STAGES);
        for (int it = 0; it < pre; ++it) {
            const uint32_t full = smem_addr(&bars[it]);
            mbar_expect_tx(issue, full, Cfg::STAGE_BYTES);
            tma_load_2d(issue && FF_GEMM_LOADS(it), smem_addr(tiles + (size_t)it * Cfg::STAGE_BYTES), &map_w, (kb0 + it) * BK,
                        n0, full);
        }
        grid_dependency_wait();
        for (int it = 0; it < pre; ++it) {
            tma_load_2d(issue && FF_GEMM_LOADS(it), smem_addr(tiles + (size_t)it * Cfg::STAGE_BYTES + Cfg::A_BYTES), &map_x,
                        (kb0 + it) * BK, t0, smem_addr(&bars[it]));
            issued = it + 1;
        }
        for (int it = pre; it < n_iters; ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            if (!__all_sync(0xffffffffu, mbar_wait(smem_addr(&bars[STAGES + s]), ph ^ 1, a.status, abort_flag, 101))) break;
            const uint32_t full = smem_addr(&bars[s]);
            mbar_expect_tx(issue, full, Cfg::STAGE_BYTES);
            unsigned char* st = tiles + (size_t)s * Cfg::STAGE_BYTES;
            tma_load_2d(issue && FF_GEMM_LOADS(it), smem_addr(st), &map_w, (kb0 + it) * BK, n0, full);
            tma_load_2d(issue && FF_GEMM_LOADS(it), smem_addr(st + Cfg::A_BYTES), &map_x, (kb0 + it) * BK, t0, full);
            issued = it + 1;
        }
        if (*abort_flag) {
            // let the copies that are still in flight land before the block's memory goes away
            for (int it = max(0, issued - STAGES); it < issued; ++it) {
                const unsigned long long start = clock64();
                while (!mbar_try_wait(smem_addr(&bars[it % STAGES]), (it / STAGES) & 1))
                    if (clock64() - start > WAIT_LIMIT_CYCLES) break;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer ----------
        const uint32_t idesc = instr_desc(TOK);
        bool ok = true;
        for (int it = 0; it < n_iters && ok; ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            ok = __all_sync(0xffffffffu, mbar_wait(smem_addr(&bars[s]), ph, a.status, abort_flag, 102));
            if (!ok) break;
            tc_fence_after();
            const uint32_t sa = smem_addr(tiles + (size_t)s * Cfg::STAGE_BYTES);
            const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
                const uint64_t da = smem_desc_sw128(sa + k * UMMA_K * 2);
                const uint64_t db = smem_desc_sw128(sb + k * UMMA_K * 2);
                tc_mma_bf16(issue, tmem_base, da, db, idesc, (it > 0 || k > 0) ? 1u : 0u);
            }
            tc_commit(issue, smem_addr(&bars[STAGES + s]));      // stage free when these MMAs have read it
            __syncwarp();
        }
        tc_commit(issue, smem_addr(&bars[2 * STAGES]));          // accumulator complete
    } else if (warp >= 2) {
        // ------------------------------------------------ epilogue ------------
        const int quad = warp & 3;                              // this warp's 32 lanes of tensor memory
        const int row = quad * 32 + lane;                       // weight row within the tile
        const int n = n0 + row;
        bool ok = true;
        if (a.ssq_in) {
            // 1/rms of the tile's tokens from the per-tile sums of squares the product in front left:
            // done while the main loop runs (these warps have nothing else to do until it ends)
            grid_dependency_wait();
            const int et = threadIdx.x - 64;
            for (int c = et; c < TOK; c += 128) {
                const int t = t0 + c;
                float ss = 0.f;
                if (t < a.T) {
#pragma unroll 8
                    for (int p = 0; p < a.ssq_parts; ++p) ss += __ldcg(a.ssq_in + (size_t)p * a.T + t);   // fixed order
                }
                s_inv[c] = 1.0f / sqrtf(ss / (float)a.norm_dim + a.norm_eps);
            }
        }
        if (a.epilogue == EPI_RESIDUAL_ADD) {
            grid_dependency_wait();                             // the residual may still be in use by the kernel before
            int c_begin = 0, c_end = TOK;
            if (a.splits > 1) {
                const int per = (TOK + a.splits - 1) / a.splits;
                c_begin = min(TOK, (int)blockIdx.z * per);
                c_end = min(TOK, c_begin + per);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int t = t0 + c_begin + i;
                res_pre[i] = (c_begin + i < c_end && t < a.T && n < a.N)
                                 ? __ldcg(reinterpret_cast<const float*>(a.out) + (size_t)t * a.ldo + n) : 0.f;
            }
            if (a.xw_out && n < a.N) wn_pre = __ldg(a.xw_w + n);
        }
        if (n_iters > 0) ok = mbar_wait(smem_addr(&bars[2 * STAGES]), 0, a.status, abort_flag, 103);
        ok = __all_sync(0xffffffffu, ok);                       // the tensor-memory loads below are warp-wide
        tc_fence_after();
        if (a.splits > 1) {
            // this block's partial tile -> its own shared memory (the pipeline's stages are
            // free now), laid out [token][row]
            float* mine = reinterpret_cast<float*>(tiles);
#pragma unroll 1
            for (int c0 = 0; c0 < TOK; c0 += 16) {
                float v[16];
                if (n_iters > 0 && ok) tc_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + c0, v);
                else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = 0.f;
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) mine[(c0 + i) * BN + row] = v[i];
            }
        }
    }
    if (a.splits > 1) cluster_sync_all();          // every block's partial tile is in place
    if (warp >= 2) {
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int n = n0 + row;
        asm volatile("bar.sync 1, 128;" ::: "memory");   // all four warps see the same abort flag below
        const bool ok = !*abort_flag;
        grid_dependency_wait();                    // the output may still be in use by the kernel before
        // tokens of the tile this block finishes: all of them without a split, else a slice
        int c_begin = 0, c_end = TOK;
        if (a.splits > 1) {
            const int per = (TOK + a.splits - 1) / a.splits;
            c_begin = min(TOK, (int)blockIdx.z * per);
            c_end = min(TOK, c_begin + per);
        }
        const uint32_t mine_addr = smem_addr(tiles);
#pragma unroll 1
        for (int c0 = c_begin; c0 < c_end; c0 += 16) {
            float v[16];
            const int cn = min(16, c_end - c0);
            if (a.splits == 1) {
                if (n_iters > 0 && ok) tc_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + c0, v);
                else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = 0.f;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = 0.f;
                // peers in a fixed order: the sum is reproducible.  Loads are issued in batches of 32
                // before the first of them is used (a load from another block's shared memory takes about
                // as long as one from the L2 cache, and one after the other they would add up): all
                // peers at once when the slice has at most four tokens, else two peers at a time.
                if (cn <= 4) {
                    float p[8][4];
#pragma unroll
                    for (int z = 0; z < 8; ++z) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const uint32_t addr = mine_addr + (uint32_t)((c0 + i) * BN + row) * 4u;
                            p[z][i] = (z < a.splits && i < cn) ? ld_peer_smem(addr, (uint32_t)z) : 0.f;
                        }
                    }
#pragma unroll
                    for (int z = 0; z < 8; ++z) {
                        if (z < a.splits) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) v[i] += p[z][i];
                        }
                    }
                } else {
                    for (int z = 0; z < a.splits; z += 2) {
                        float p0[16], p1[16];
                        const bool two = z + 1 < a.splits;
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const uint32_t addr = mine_addr + (uint32_t)((c0 + i) * BN + row) * 4u;
                            p0[i] = i < cn ? ld_peer_smem(addr, (uint32_t)z) : 0.f;
                            p1[i] = (two && i < cn) ? ld_peer_smem(addr, (uint32_t)(z + 1)) : 0.f;
                        }
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            v[i] += p0[i];
                            if (two) v[i] += p1[i];
                        }
                    }
                }
            }
            if (!ok) continue;
            if (a.ssq_in) {
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] *= s_inv[min(c0 + i, TOK - 1)];
            }
            if (a.epilogue == EPI_SWIGLU) {
                // rows come in groups of 32: 16 gate rows, then the 16 up rows of the same columns
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float other = __shfl_xor_sync(0xffffffffu, v[i], 16);
                    const int t = t0 + c0 + i;
                    const int col = (n0 + quad * 32) / 2 + lane;
                    if (i < cn && lane < 16 && t < a.T && col < a.N / 2) {
                        const float g = v[i];
                        reinterpret_cast<bf16*>(a.out)[(size_t)t * a.ldo + col] =
                            __float2bfloat16_rn(g / (1.0f + expf(-g)) * other);
                    }
                }
            } else if (a.epilogue == EPI_RESIDUAL_ADD && a.xw_out) {
                // out += acc; and for the norm that follows: bfloat16(out * w) and this tile's sums of squares
                const float wn = wn_pre;
                const bool first = c0 == c_begin;               // its residual values are in registers already
                float sq[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int t = t0 + c0 + i;
                    sq[i] = 0.f;
                    if (i >= cn || t >= a.T || n >= a.N) continue;
                    const size_t o = (size_t)t * a.ldo + n;
                    const float r = (first ? res_pre[i] : reinterpret_cast<float*>(a.out)[o]) + v[i];
                    reinterpret_cast<float*>(a.out)[o] = r;
                    a.xw_out[(size_t)t * a.N + n] = __float2bfloat16_rn(r * wn);
                    sq[i] = r * r;
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float w_sum = warp_sum(sq[i]);
                    if (lane == 0) s_red[quad][i] = w_sum;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const int et = threadIdx.x - 64;
                if (et < cn && t0 + c0 + et < a.T)
                    a.ssq_out[(size_t)blockIdx.x * a.T + t0 + c0 + et] =
                        s_red[0][et] + s_red[1][et] + s_red[2][et] + s_red[3][et];
                asm volatile("bar.sync 1, 128;" ::: "memory");
            } else if (n < a.N) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int t = t0 + c0 + i;
                    if (i >= cn || t >= a.T) continue;
                    const size_t o = (size_t)t * a.ldo + n;
                    if (a.epilogue == EPI_BF16) reinterpret_cast<bf16*>(a.out)[o] = __float2bfloat16_rn(v[i]);
                    else if (a.epilogue == EPI_F32) reinterpret_cast<float*>(a.out)[o] = v[i];
                    else reinterpret_cast<float*>(a.out)[o] = (c0 == c_begin ? res_pre[i] : reinterpret_cast<float*>(a.out)[o]) + v[i];
                }
            }
        }
    }
    if (a.splits > 1) cluster_sync_all();          // peers may still be reading this block's tile
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
    }
}

template <int TOK>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& a_in, int n_tiles, int t_tiles,
                  int pdl, cudaStream_t stream) {
    using Cfg = TileCfg<TOK>;
    FF_SMEM_LIMIT(gemm_tc_kernel<TOK>, Cfg::smem(Cfg::DEEP));
    GemmArgs a = a_in;
    const long long blocks = (long long)n_tiles * t_tiles * a.splits;
    // half an SM's shared memory per block: the next product's blocks can move in beside this one's and
    // request their first weight tiles while this one is still running
    (void)blocks;
    a.stages = Cfg::SHALLOW;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tiles, t_tiles, a.splits);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = Cfg::smem(a.stages);
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    int na = 0;
    if (a.splits > 1) {                         // the K ranges of a tile form one cluster
        attrs[na].id = cudaLaunchAttributeClusterDimension;
        attrs[na].val.clusterDim.x = 1;
        attrs[na].val.clusterDim.y = 1;
        attrs[na].val.clusterDim.z = a.splits;
        ++na;
    }
    if (pdl || g_ff_pdl) {
        attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<TOK>, mw, mx, a);
    if (e != cudaSuccess) return (int)e;
    return 0;
}

}  // namespace ff

using namespace ff;

// Tokens per tile and K ranges (= blocks per cluster, at most 8) a call would use.
FF_EXPORT int ff_gemm_tc_plan(int T, int N, int K, int want_splits, int* tok_out, int* splits_out) {
    int tok = 16;
    while (tok < T && tok < 256) tok <<= 1;
    const int num_kb = (K + BK - 1) / BK;
    int splits = want_splits < 1 ? 1 : want_splits;
    if (splits > 8) splits = 8;
    if (tok > 64) splits = 1;                            // large token tiles have enough blocks without
    if (splits > num_kb) splits = num_kb;
    const int per = (num_kb + splits - 1) / splits;
    splits = (num_kb + per - 1) / per;                   // no empty K range
    *tok_out = tok;
    *splits_out = splits;
    return 0;
}

// x: bfloat16 [T, K] contiguous; w: bfloat16 [N, K] contiguous; K a multiple of 8.
// epilogue: 0 bf16 out [T, ldo], 1 f32 out, 2 f32 out += , 3 swiglu (bf16 out [T, ldo], N/2 columns).
// pdl: launch with programmatic stream serialization (the kernel before must tolerate an early start
// of this one, which only prefetches weights before it waits).
// Norm folded in (all optional, see GemmArgs): xw_out/xw_w/ssq_out with EPI_RESIDUAL_ADD
// (ssq_out holds ceil(N/128) * T floats); ssq_in/ssq_parts/norm_dim/norm_eps on the consuming side.
FF_EXPORT int ff_gemm_tc(const void* x, const void* w, void* out, int ldo, int T, int N, int K, int epilogue,
                         int want_splits, int pdl, void* xw_out, const float* xw_w, float* ssq_out,
                         const float* ssq_in, int ssq_parts, int norm_dim, float norm_eps, int* status,
                         cudaStream_t stream) {
    if (xw_out && (epilogue != EPI_RESIDUAL_ADD || !xw_w || !ssq_out)) return FF_ERR_BAD_ARG;
    if (ssq_in && (ssq_parts <= 0 || norm_dim <= 0)) return FF_ERR_BAD_ARG;
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0 || (K % 8) || epilogue < 0 || epilogue > 3) return FF_ERR_BAD_ARG;
    if (epilogue == EPI_SWIGLU && (N % 32)) return FF_ERR_UNSUPPORTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return FF_ERR_BAD_ARG;
    int tok, splits;
    ff_gemm_tc_plan(T, N, K, want_splits, &tok, &splits);
    const int n_tiles = (N + BN - 1) / BN, t_tiles = (T + tok - 1) / tok;
    const int num_kb = (K + BK - 1) / BK;
    CUtensorMap mw, mx;
    int rc = make_map(w, N, K, BN, &mw);
    if (rc) return rc;
    rc = make_map(x, T, K, tok, &mx);
    if (rc) return rc;
    GemmArgs a;
    a.out = out; a.ldo = ldo; a.T = T; a.N = N; a.K = K; a.epilogue = epilogue; a.splits = splits;
    a.kb_per_split = (num_kb + splits - 1) / splits;
    a.status = status;
    a.xw_out = (bf16*)xw_out; a.xw_w = xw_w; a.ssq_out = ssq_out;
    a.ssq_in = ssq_in; a.ssq_parts = ssq_parts; a.norm_dim = norm_dim; a.norm_eps = norm_eps;
    switch (tok) {
        case 16: return launch<16>(mw, mx, a, n_tiles, t_tiles, pdl, stream);
        case 32: return launch<32>(mw, mx, a, n_tiles, t_tiles, pdl, stream);
        case 64: return launch<64>(mw, mx, a, n_tiles, t_tiles, pdl, stream);
        case 128: return launch<128>(mw, mx, a, n_tiles, t_tiles, pdl, stream);
        default: return launch<256>(mw, mx, a, n_tiles, t_tiles, pdl, stream);
    }
}
