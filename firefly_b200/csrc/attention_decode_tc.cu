// Split-KV attention for decode steps (one token per sequence) on the fifth-generation tensor
// cores, written as a streamer of the cache: keys and values are the large operands.
//
// A block owns one (sequence, kv head, range of keys).  The group's G <= 16 query heads are the
// small operand, so the products are taken transposed, with the keys (then the head dimension) as
// the 128 rows of the MMA:
//   S^T = K Q^T      M = 128 keys of a tile, N = 16 query rows, K = head size; K tile as it lies in
//                    the cache pages (brought in by TMA), Q^T from shared memory; S^T (128 x 16,
//                    float32) in tensor memory, two buffers;
//   softmax          four warps, one thread per key: its 16 scores, p = 2^(s*scale - m) against a
//                    reference maximum per query row that all threads hold alike and move only
//                    when some score exceeds it by more than 2^8 (a vote over the block, then a
//                    reduction; rare after the first tile); P^T as bfloat16 into shared memory;
//   O^T += V^T P^T   M = 128 = head size, N = 16, K = 128 keys; V^T is the V tile as it lies in
//                    the pages (the M-major operand form), O^T (128 x 16, float32) in tensor memory.
// Three stages of (K, V) tiles of 128 keys (64 KB each) keep up to 192 KB of the cache in flight
// per SM; one warp starts the page copies (a lane per box), one warp issues the MMAs.  Tiles that
// cannot hold the newest key are requested before the wait for the kernel in front (which
// produces q and that key only).  With one range the output is final; else partial (o, m, l) go
// to scratch memory for attn_combine_kernel (attention_mma.cu), in the same convention.
//
// Head size 128 only (the head dimension is the M of the second product); pages of 8 to 64 tokens;
// groups of at most 16 query heads.  Other sizes run attn_decode_kernel (mma.sync), which this
// kernel replaces where it applies; the reference's decode kernel is a scalar loop over the pages
// (src/kernels/attention.cu:288-446).
// Every mbarrier wait is bounded; on time-out the kernel records code 109 in the status word,
// stops, frees its tensor memory and returns.
//
// Cache layout of a slot: [num_blocks][2 (k,v)][n_kv_heads][block_size][128].
#include "common.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>
#include <math_constants.h>

#include <cstring>
#include <mutex>
#include <unordered_map>

namespace ff {

constexpr int D = 128;                  // head size = rows of the second product
constexpr int BN = 128;                 // keys per tile = rows of the first product
constexpr int NQ = 16;                  // query rows (padded group)
constexpr int STAGES = 3;
constexpr int ADT_THREADS = 192;        // warps 0-3 softmax, warp 4 loads, warp 5 MMAs
constexpr float LOG2E = 1.4426950408889634f;
constexpr unsigned long long WAIT_LIMIT_CYCLES = 2000000000ull;

constexpr int TILE_BYTES = BN * D * 2;          // one K or V tile: 2 panels x [128 rows][128 B]
constexpr int Q_BYTES = NQ * D * 2;             // 2 panels x [16 rows][128 B]
constexpr int P_BYTES = NQ * BN * 2;            // 2 panels (64 keys each) x [16 rows][128 B]
constexpr int TMEM_COLS = 64;                   // S^T two buffers of 16 columns, O^T 16 columns
constexpr int MAX_PAGE_LIST = 2048;     // page ids of a block's tiles kept in shared memory (longer ranges look them up per tile)
constexpr size_t ADT_SMEM = 1024 + (size_t)STAGES * 2 * TILE_BYTES + Q_BYTES + 2 * P_BYTES + 256 + MAX_PAGE_LIST * 4;

enum { B_KV_FULL = 0, B_KV_EMPTY = 3, B_S_FULL = 6, B_P_FULL = 8, B_PV_DONE = 10, B_Q_READY = 11, B_COUNT = 12 };

__device__ __forceinline__ uint32_t sa(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mb_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mb_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mb_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mb_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred P1;\n\tmbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
                 "selp.b32 %0, 1, 0, P1;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mb_wait(uint32_t bar, uint32_t parity, int* status, volatile int* abort_flag) {
    const unsigned long long start = clock64();
    uint32_t spins = 0;
    while (!mb_try(bar, parity)) {
        __nanosleep(32);
        if (((++spins) & 1023u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - start > WAIT_LIMIT_CYCLES) {
                atomicExch(status, 109);
                *abort_flag = 1;
                return false;
            }
        }
    }
    return true;
}
__device__ __forceinline__ void tma_2d(uint32_t dst, const void* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tc_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// `issue` is true in the one lane of the converged MMA warp that acts
__device__ __forceinline__ void tc_commit_to(bool issue, uint32_t bar) {
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
                 "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
                 ::"r"(bar), "r"((uint32_t)issue) : "memory");
}
__device__ __forceinline__ void tc_mma(bool issue, uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                 "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(acc), "r"((uint32_t)issue) : "memory");
}
__device__ __forceinline__ void tm_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tm_st16(uint32_t taddr, const float (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
                   "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
                   "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])),
                   "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
                   "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
                   "r"(__float_as_uint(v[15])) : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {   // 2^x; -inf -> 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Barrier over the 128 softmax threads that also ORs a predicate: every thread gets the same answer.
__device__ __forceinline__ bool bar_or_128(bool pred) {
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %1, 0;\n\tbarrier.cta.red.or.pred q, 1, 128, p;\n\t"
                 "selp.b32 %0, 1, 0, q;\n\t}" : "=r"(r) : "r"((uint32_t)pred) : "memory");
    return r != 0;
}
__device__ __forceinline__ void bar_128() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Operand descriptors.  Tiles are made of 64-column panels whose 128-byte rows are swizzled in groups
// of eight (the layout TMA writes with the 128-byte swizzle).
// K-major (the reduction dimension runs along the 128-byte row): groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// M-major (the rows of the tile are the reduction dimension, the 128-byte row runs along M): groups of 8
// reduction rows 1024 bytes apart (stride offset), 64-column panels `panel_bytes` apart (leading offset).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t panel_bytes) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)((panel_bytes >> 4) & 0x3FFF) << 16) |
           ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// bfloat16 x bfloat16 -> float32, M = 128, N = 16; a_m_major: the A operand is M-major
__device__ __forceinline__ uint32_t idesc_bf16(bool a_m_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((a_m_major ? 1u : 0u) << 15) | ((uint32_t)(NQ >> 3) << 17) |
           ((uint32_t)(128 >> 4) << 24);
}

struct alignas(64) TensorMapArg { unsigned char bytes[128]; };   // a CUtensorMap, opaque to device code

__global__ void __launch_bounds__(ADT_THREADS)
attn_dec_tc_kernel(const __grid_constant__ TensorMapArg kv_map, const bf16* __restrict__ q, int q_stride,
                   const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_q,
                   const int* __restrict__ ctx_lens, bf16* __restrict__ out, int out_stride,
                   float* __restrict__ part_o, float* __restrict__ part_ml, int nq, int nkv, int block_size,
                   int num_blocks, float scale_log2, int window, int num_splits, int* __restrict__ status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* KV = base;                                        // [stage][K|V][2 panels][128][128 B]
    unsigned char* Qs = KV + (size_t)STAGES * 2 * TILE_BYTES;        // [2 panels][16][128 B]
    unsigned char* Ps = Qs + Q_BYTES;                                // [2 buffers][2 panels][16][128 B]
    uint64_t* bars = reinterpret_cast<uint64_t*>(Ps + 2 * P_BYTES);
    int* s_pages = reinterpret_cast<int*>(bars + 32);
    __shared__ int s_abort;
    __shared__ uint32_t s_tmem;
    __shared__ float s_red[4][NQ];                                   // per-warp maxima / sums of the query rows
    const int G = nq / nkv;
    const int seq = blockIdx.x, kh = blockIdx.y, split = blockIdx.z;
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    volatile int* abort_flag = &s_abort;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int i = 0; i < B_COUNT; ++i) mb_init(sa(&bars[i]), (i == B_P_FULL || i == B_P_FULL + 1 || i == B_Q_READY) ? 4 : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(sa(&s_tmem)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // the step's metadata does not depend on the kernel in front
    const int tok = cu_q[seq];
    const int pos = ctx_lens[seq];
    const int kv_hi = pos + 1;
    const int kv_lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* bt = block_table + (size_t)seq * max_blocks;
    const int t0 = kv_lo / BN, t1 = (kv_hi + BN - 1) / BN;
    const int per = (t1 - t0 + num_splits - 1) / num_splits;
    const int t_begin = t0 + split * per, t_end = min(t1, t_begin + per);
    const int n_tiles = max(0, t_end - t_begin);
    const int pages_per_tile = BN / block_size;
    tc_before();
    __syncthreads();
    tc_after();
    const uint32_t tmem = s_tmem;
    const uint32_t tm_S = tmem;                  // two buffers: columns [0, 16) and [16, 32)
    const uint32_t tm_O = tmem + 2 * NQ;         // columns [32, 48)

    if (warp < 4) {
        // ------------------------------------------------ softmax, one thread per key (later: per d) --
        const int r = threadIdx.x;                            // key within a tile; head-dimension index in O^T
        const uint32_t lane_base = (uint32_t)((warp * 32) << 16);
        // zero Q's rows beyond the group and the P buffers once (finite numbers for the padded rows)
        for (int i = threadIdx.x; i < (Q_BYTES + 2 * P_BYTES) / 16; i += 128)
            reinterpret_cast<uint4*>(Qs)[i] = make_uint4(0u, 0u, 0u, 0u);
        bar_128();
        asm volatile("griddepcontrol.wait;" ::: "memory");
        // q rows of the group -> the swizzled Q tile: 16 chunks of 16 bytes a row, G rows
        for (int c = threadIdx.x; c < G * (D / 8); c += 128) {
            const int row = c / (D / 8), ch = c % (D / 8);
            const uint4 v = *reinterpret_cast<const uint4*>(q + (size_t)tok * q_stride + (size_t)(kh * G + row) * D + ch * 8);
            *reinterpret_cast<uint4*>(Qs + (ch >> 3) * (NQ * 128) + row * 128 + (((ch & 7) ^ (row & 7)) << 4)) = v;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mb_arrive(sa(&bars[B_Q_READY]));

        float m[NQ], l[NQ];
#pragma unroll
        for (int n = 0; n < NQ; ++n) { m[n] = -CUDART_INF_F; l[n] = 0.f; }
        bool failed = false;
        for (int j = 0; j < n_tiles; ++j) {
            if (!failed) failed = !__all_sync(0xffffffffu, mb_wait(sa(&bars[B_S_FULL + (j & 1)]), (j >> 1) & 1, status, abort_flag));
            float s[NQ];
            const int key = (t_begin + j) * BN + r;
            const bool visible = key >= kv_lo && key < kv_hi;
            bool grow = false;
            if (!failed) {
                tc_after();
                tm_ld16(tm_S + (uint32_t)((j & 1) * NQ) + lane_base, s);
#pragma unroll
                for (int n = 0; n < NQ; ++n) {
                    s[n] = visible ? s[n] * scale_log2 : -CUDART_INF_F;
                    grow = grow || s[n] > m[n] + 8.0f;                 // also true while m is -inf and s is not
                }
            }
            // does any thread see a score far above the reference?  (the barrier also tells every
            // warp whether one has given up, so that all leave together)
            const bool stop = bar_or_128(failed || *abort_flag != 0);
            if (stop) { failed = true; break; }
            const bool move = bar_or_128(grow);
            float corr[NQ];
#pragma unroll
            for (int n = 0; n < NQ; ++n) corr[n] = 1.0f;
            if (move) {
                // the reference maxima follow the tile's column maxima (over all 128 keys)
#pragma unroll
                for (int n = 0; n < NQ; ++n) {
                    float v = s[n];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
                    if (lane == 0) s_red[warp][n] = v;
                }
                bar_128();
#pragma unroll
                for (int n = 0; n < NQ; ++n) {
                    const float cm = fmaxf(fmaxf(s_red[0][n], s_red[1][n]), fmaxf(s_red[2][n], s_red[3][n]));
                    const float m_new = fmaxf(m[n], cm);
                    corr[n] = m[n] == -CUDART_INF_F ? 0.f : fast_exp2(m[n] - m_new);    // m_new finite here or both -inf
                    if (m_new == -CUDART_INF_F) corr[n] = 1.0f;
                    m[n] = m_new;
                    l[n] *= corr[n];
                }
                bar_128();                                              // s_red may be written again
            }
            // p = 2^(s - m) as bfloat16 into P^T [query row][key]; the sums add the rounded values
            unsigned char* Pt = Ps + (j & 1) * P_BYTES + (r >> 6) * (NQ * 128);
            const int kc = r & 63;                                      // key within its 64-key panel
#pragma unroll
            for (int n = 0; n < NQ; ++n) {
                const float p = m[n] == -CUDART_INF_F ? 0.f : fast_exp2(s[n] - m[n]);
                const bf16 pb = __float2bfloat16_rn(p);
                l[n] += __bfloat162float(pb);
                *reinterpret_cast<bf16*>(Pt + n * 128 + ((((kc >> 3) ^ (n & 7)) << 4) | ((kc & 7) << 1))) = pb;
            }
            if (move && j > 0) {
                // O^T is complete once the last P V is done; thread = head-dimension index, 16 query rows
                if (!__all_sync(0xffffffffu, mb_wait(sa(&bars[B_PV_DONE]), (j - 1) & 1, status, abort_flag))) {
                    failed = true;
                    continue;
                }
                tc_after();
                float o[NQ];
                tm_ld16(tm_O + lane_base, o);
#pragma unroll
                for (int n = 0; n < NQ; ++n) o[n] *= corr[n];
                tm_st16(tm_O + lane_base, o);
                tc_before();
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mb_arrive(sa(&bars[B_P_FULL + (j & 1)]));
        }
        // ------------------------------------------------ epilogue ------------
        if (n_tiles > 0 && !failed)
            failed = !__all_sync(0xffffffffu, mb_wait(sa(&bars[B_PV_DONE]), (n_tiles - 1) & 1, status, abort_flag));
        // the row sums over all 128 keys' threads
#pragma unroll
        for (int n = 0; n < NQ; ++n) {
            float v = l[n];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) s_red[warp][n] = v;
        }
        const bool stop = bar_or_128(failed || *abort_flag != 0);
        if (!stop) {
            float o[NQ];
            if (n_tiles > 0) {
                tc_after();
                tm_ld16(tm_O + lane_base, o);
            } else {
#pragma unroll
                for (int n = 0; n < NQ; ++n) o[n] = 0.f;
            }
#pragma unroll
            for (int n = 0; n < NQ; ++n) {
                if (n >= G) continue;
                const float L = (s_red[0][n] + s_red[1][n]) + (s_red[2][n] + s_red[3][n]);
                const int head = kh * G + n;
                if (num_splits == 1) {
                    out[(size_t)tok * out_stride + (size_t)head * D + r] = __float2bfloat16_rn(o[n] / L);
                } else {
                    const size_t p = ((size_t)seq * nq + head) * num_splits + split;
                    part_o[p * D + r] = o[n];
                    if (r == 0) { part_ml[p * 2] = m[n]; part_ml[p * 2 + 1] = L; }
                }
            }
        }
    } else if (warp == 4) {
        // ------------------------------------------------ loads: K and V tiles by TMA --
        // A tile is pages_per_tile pages x (K, V) x 2 panels = boxes of block_size rows; a lane per box.
        // Tiles that end before the newest key are requested before the wait for the kernel in front.
        const int boxes = pages_per_tile * 4;
        // the page ids of all tiles first (they do not depend on the kernel in front): -1 where no
        // page is to be loaded
        const int n_list = n_tiles * pages_per_tile;
        const bool listed = n_list <= MAX_PAGE_LIST;
        auto page_of = [&](int j, int p) -> int {
            const int first_key = ((t_begin + j) * BN) + p * block_size;
            const int pi = first_key / block_size;
            int page = -1;
            if (first_key < kv_hi && first_key + block_size > kv_lo && pi < max_blocks) page = bt[pi];
            return page >= num_blocks ? -1 : page;
        };
        if (listed) {
            for (int i = lane; i < n_list; i += 32) s_pages[i] = page_of(i / pages_per_tile, i % pages_per_tile);
            __syncwarp();
        }
        bool waited = false;
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int s = j % STAGES;
            const int key0 = (t_begin + j) * BN;
            if (!waited && key0 + BN > pos) {
                asm volatile("griddepcontrol.wait;" ::: "memory");
                waited = true;
            }
            ok = __all_sync(0xffffffffu, mb_wait(sa(&bars[B_KV_EMPTY + s]), ((j / STAGES) & 1) ^ 1, status, abort_flag));
            if (!ok) break;
            const uint32_t bar = sa(&bars[B_KV_FULL + s]);
            unsigned char* st = KV + (size_t)s * 2 * TILE_BYTES;
            // Pass 1: V boxes that no page is loaded into are zeroed (0 x stale bits could be NaN in the
            // second product; absent K rows only give scores that the softmax masks), and the boxes are
            // counted.  Pass 2: the copies.
            int n_valid = 0;
            for (int b0 = 0; b0 < boxes; b0 += 32) {
                const int b = b0 + lane;
                int page = -1;
                if (b < boxes) {
                    const int p = b >> 2, kv = (b >> 1) & 1, h = b & 1;
                    page = listed ? s_pages[j * pages_per_tile + p] : page_of(j, p);
                    if (page < 0 && kv == 1) {
                        uint4* z = reinterpret_cast<uint4*>(st + TILE_BYTES + h * (BN * 128) + p * block_size * 128);
                        for (int i = 0; i < block_size * 8; ++i) z[i] = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                n_valid += __popc(__ballot_sync(0xffffffffu, page >= 0));
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mb_expect_tx(bar, (uint32_t)(n_valid * block_size * 128));
            __syncwarp();
            for (int b0 = 0; b0 < boxes; b0 += 32) {
                const int b = b0 + lane;
                if (b >= boxes) continue;
                const int p = b >> 2, kv = (b >> 1) & 1, h = b & 1;
                const int page = listed ? s_pages[j * pages_per_tile + p] : page_of(j, p);
                if (page < 0) continue;
                const int y = ((page * 2 + kv) * nkv + kh) * block_size;
                tma_2d(sa(st + kv * TILE_BYTES + h * (BN * 128) + p * block_size * 128), &kv_map, h * 64, y, bar);
            }
        }
        if (!waited) asm volatile("griddepcontrol.wait;" ::: "memory");
    } else if (warp == 5) {
        // ------------------------------------------------ MMAs -----------------
        const uint32_t idesc_qk = idesc_bf16(false);
        const uint32_t idesc_pv = idesc_bf16(true);
        const bool issue = lane == 0;
        bool ok = n_tiles == 0 || mb_wait(sa(&bars[B_Q_READY]), 0, status, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        tc_after();
        auto issue_qk = [&](int j) -> bool {
            const int s = j % STAGES;
            if (!__all_sync(0xffffffffu, mb_wait(sa(&bars[B_KV_FULL + s]), (j / STAGES) & 1, status, abort_flag))) return false;
            tc_after();
            const uint32_t ks = sa(KV + (size_t)s * 2 * TILE_BYTES);
#pragma unroll
            for (int k = 0; k < D / 16; ++k) {
                const uint64_t da = desc_k_major(ks + (k >> 2) * (BN * 128) + (k & 3) * 32);
                const uint64_t db = desc_k_major(sa(Qs) + (k >> 2) * (NQ * 128) + (k & 3) * 32);
                tc_mma(issue, tm_S + (uint32_t)((j & 1) * NQ), da, db, idesc_qk, k > 0 ? 1u : 0u);
            }
            tc_commit_to(issue, sa(&bars[B_S_FULL + (j & 1)]));
            __syncwarp();
            return true;
        };
        if (ok && n_tiles > 0) ok = issue_qk(0);
        for (int j = 0; j < n_tiles && ok; ++j) {
            if (j + 1 < n_tiles) {
                ok = issue_qk(j + 1);
                if (!ok) break;
            }
            const int s = j % STAGES;
            ok = __all_sync(0xffffffffu, mb_wait(sa(&bars[B_P_FULL + (j & 1)]), (j >> 1) & 1, status, abort_flag));
            if (!ok) break;
            tc_after();
            const uint32_t vs = sa(KV + (size_t)s * 2 * TILE_BYTES + TILE_BYTES);
            const uint32_t ps = sa(Ps + (j & 1) * P_BYTES);
#pragma unroll
            for (int k = 0; k < BN / 16; ++k) {
                const uint64_t da = desc_mn_major(vs + k * 16 * 128, BN * 128);
                const uint64_t db = desc_k_major(ps + (k >> 2) * (NQ * 128) + (k & 3) * 32);
                tc_mma(issue, tm_O, da, db, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
            }
            tc_commit_to(issue, sa(&bars[B_PV_DONE]));
            tc_commit_to(issue, sa(&bars[B_KV_EMPTY + s]));
            __syncwarp();
        }
    }
    tc_before();
    __syncthreads();
    if (warp == 5) {
        __syncwarp();
        tc_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------ host side --
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Tensor map of a cache slot seen as [rows, 128] bfloat16: boxes of block_size rows x 64 columns, 128-byte swizzle.
static int cache_map(const void* cache, long long rows, int block_size, CUtensorMap* out) {
    struct Key { const void* p; long long rows; int bs; };
    static std::mutex mu;
    static std::unordered_map<const void*, std::pair<Key, CUtensorMap>> cache_maps;
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache_maps.find(cache);
    if (it != cache_maps.end() && it->second.first.rows == rows && it->second.first.bs == block_size) {
        *out = it->second.second;
        return 0;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return FF_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)block_size};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return FF_ERR_BAD_ARG;
    if (cache_maps.size() > 4096) cache_maps.clear();
    cache_maps[cache] = {Key{cache, rows, block_size}, *out};
    return 0;
}

}  // namespace ff

using namespace ff;

// Every sequence has exactly one token; head size 128.  part_o: float [n_seqs*nq*num_splits*128],
// part_ml: float [n_seqs*nq*num_splits*2] (unused when num_splits == 1).  With more than one range the
// caller joins the partial results with attn_combine_kernel's entry (ff_attn_combine).
FF_EXPORT int ff_attn_dec_tc(const void* q, int q_stride, const void* cache, const int* block_table, int max_blocks,
                             const int* cu_q, const int* ctx_lens, int n_seqs, void* out, int out_stride,
                             float* part_o, float* part_ml, int nq, int nkv, int block_size, int num_blocks,
                             float scale, int window, int num_splits, int* status, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (nkv <= 0 || nq % nkv || num_splits < 1) return FF_ERR_BAD_ARG;
    if (nq / nkv > NQ) return FF_ERR_UNSUPPORTED;
    if (block_size < 8 || block_size > 64 || (block_size & (block_size - 1))) return FF_ERR_UNSUPPORTED;
    if (((uintptr_t)cache & 127) || ((uintptr_t)q & 15) || (q_stride % 8)) return FF_ERR_UNSUPPORTED;
    const long long rows = (long long)num_blocks * 2 * nkv * block_size;
    if (rows >= (1ll << 31) || n_seqs > 65535 * 32 || nkv > 65535 || num_splits > 65535) return FF_ERR_UNSUPPORTED;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn_dec_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ADT_SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    CUtensorMap map;
    int rc = cache_map(cache, rows, block_size, &map);
    if (rc) return rc;
    TensorMapArg arg;
    std::memcpy(arg.bytes, &map, sizeof(map));
    FF_LAUNCH((attn_dec_tc_kernel), dim3(n_seqs, nkv, num_splits), ADT_THREADS, ADT_SMEM, stream, arg, (const bf16*)q,
              q_stride, block_table, max_blocks, cu_q, ctx_lens, (bf16*)out, out_stride, part_o, part_ml, nq, nkv,
              block_size, num_blocks, scale * LOG2E, window, num_splits, status);
    return 0;
}
