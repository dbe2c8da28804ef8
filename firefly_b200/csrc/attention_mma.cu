// Tensor-core attention over the paged cache for bfloat16: a tiled kernel for
// portions of prompts (and any mix of sequences), a split-KV kernel for steps in
// which every sequence decodes one token, and the kernel that joins the splits.
//
// Both kernels pack the query heads of one kv head into the rows of a tile
// (row = token * G + head-in-group, G = num_heads / num_kv_heads), so a key or
// value is fetched once for the whole group; the reference's decode kernel re-reads
// it per q head (src/kernels/attention.cu:291-447) and its prefill kernel works on
// the portion's own k and v instead of the cache (src/model/qwen_model.cu:147-151).
// Scores, running max and sum, and the output accumulator are 32-bit; q.k and p.v
// run on mma.sync m16n8k16 with bfloat16 operands.  Keys come from the pages by
// absolute position: a query at position p sees keys max(0, p-W+1)..p.
//
// Compiled once per head size: -DFF_HEAD_DIM=<multiple of 16, up to 256>.
// Cache layout of a slot: [num_blocks][2 (k,v)][n_kv_heads][block_size][head_dim].
#include "common.cuh"
#include <math_constants.h>

#ifndef FF_HEAD_DIM
#define FF_HEAD_DIM 128
#endif

namespace ff {

constexpr int D = FF_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16, at most 256");
constexpr int KSTR = D + 8;            // padded row: ldmatrix rows fall in distinct banks
constexpr int BN = 64;                 // keys per tile
constexpr int BM = 64;                 // rows per tile of the tiled kernel (4 warps x 16)
constexpr int NTHREADS = 128;
constexpr int CHUNKS = D / 8;          // 16-byte pieces per row
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;      // n = 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

static_assert(NTHREADS >= BN, "one thread looks up each key row of a tile");
static_assert((BN * CHUNKS) % NTHREADS == 0, "the copy loop has no tail");

// Where each key row of the tile that starts at key0 lies in the cache, as an element offset
// of its K row (the V row is v_off further), or -1 when the key is outside [kv_lo, kv_hi) or
// its page is missing.  Thread r < BN looks up row r: one block-table read per row and tile.
// A key that should be read but has no valid page raises status 4 (a fault of the bookkeeping: the
// row then counts as a key of zeros, and the host must not trust the step's output).
__device__ __forceinline__ long long kv_row_offset(const int* __restrict__ bt, int max_blocks, int num_blocks,
                                                   int nkv, int kh, int block_size, int key, int kv_lo, int kv_hi,
                                                   int* status) {
    long long off = -1;
    if (key >= kv_lo && key < kv_hi) {
        const int pi = key / block_size;
        const int page = pi < max_blocks ? bt[pi] : -1;
        if (page >= 0 && page < num_blocks)
            off = ((((long long)page * 2) * nkv + kh) * block_size + (key - pi * block_size)) * D;
        else if (status != nullptr)
            atomicExch(status, 4);
    }
    return off;
}
__device__ __forceinline__ void kv_row_offsets(long long* row_off, const int* __restrict__ bt, int max_blocks,
                                               int num_blocks, int nkv, int kh, int block_size, int key0,
                                               int kv_lo, int kv_hi, int* status) {
    if (threadIdx.x < BN)
        row_off[threadIdx.x] = kv_row_offset(bt, max_blocks, num_blocks, nkv, kh, block_size, key0 + threadIdx.x,
                                             kv_lo, kv_hi, status);
}

// Copy a tile's K and V rows into shared memory, 16 bytes a thread, neighbouring threads on
// neighbouring pieces of a row; rows that are not there become zeros.
__device__ __forceinline__ void load_kv_tile(bf16* Ks, bf16* Vs, const bf16* __restrict__ cache,
                                             const long long* row_off, size_t v_off) {
#pragma unroll
    for (int i = 0; i < BN * CHUNKS / NTHREADS; ++i) {
        const int idx = i * NTHREADS + threadIdx.x;
        const int row = idx / CHUNKS, ch = idx % CHUNKS;
        const long long off = row_off[row];
        const bool ok = off >= 0;
        const bf16* src = cache + (ok ? off : 0) + ch * 8;
        cp_async16(Ks + row * KSTR + ch * 8, src, ok);
        cp_async16(Vs + row * KSTR + ch * 8, src + v_off, ok);
    }
}

// One warp's attention state for 16 rows: running max / sum and the output tile.
// `KN` keys of each tile belong to this warp.
template <int KN>
struct WarpState {
    float o[D / 8][4];
    float m[2], l[2];

    __device__ __forceinline__ void init() {
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
        m[0] = m[1] = -CUDART_INF_F;
        l[0] = l[1] = 0.f;
    }

    // Qs: this warp's 16 rows of q in smem ([16][KSTR]); Ks/Vs: this warp's KN keys.
    // key0: absolute index of the warp's first key.  Row r of the fragment (g, g+8)
    // sees keys in [lo[r], hi[r]); scores are multiplied by scale_log2 (= scale*log2 e).
    __device__ __forceinline__ void step(const bf16* Qs, const bf16* Ks, const bf16* Vs, int key0,
                                         const int (&lo)[2], const int (&hi)[2], float scale_log2,
                                         bool need_mask) {
        const int lane = threadIdx.x & 31;
        float s[KN / 8][4];
#pragma unroll
        for (int j = 0; j < KN / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
        // S = Q K^T
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            uint32_t a[4];
            ldsm_x4(a, Qs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * KSTR + kk * 16 + 8 * (lane >> 4));
#pragma unroll
            for (int jj = 0; jj < KN / 16; ++jj) {
                uint32_t b[4];
                ldsm_x4(b, Ks + (jj * 16 + (lane & 7) + 8 * (lane >> 4)) * KSTR + kk * 16 + 8 * ((lane >> 3) & 1));
                mma_bf16(s[2 * jj], a, b[0], b[1]);
                mma_bf16(s[2 * jj + 1], a, b[2], b[3]);
            }
        }
        // scale, mask, running max
        const int t4 = lane & 3;
        float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
        for (int j = 0; j < KN / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = e >> 1;
                float v = s[j][e] * scale_log2;
                if (need_mask) {
                    const int key = key0 + j * 8 + 2 * t4 + (e & 1);
                    if (key < lo[r] || key >= hi[r]) v = -CUDART_INF_F;
                }
                s[j][e] = v;
                mx[r] = fmaxf(mx[r], v);
            }
        }
        float corr[2], msafe[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m[r], mx[r]);
            msafe[r] = m_new == -CUDART_INF_F ? 0.f : m_new;
            corr[r] = exp2f(m[r] - msafe[r]);      // m = -inf: 0
            m[r] = m_new;
            l[r] *= corr[r];
        }
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        // P = exp2(S - m), row sums (per thread; joined over the quad at the end)
#pragma unroll
        for (int j = 0; j < KN / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = e >> 1;
                const float p = exp2f(s[j][e] - msafe[r]);
                s[j][e] = p;
                l[r] += p;
            }
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < KN / 16; ++kk) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int nn = 0; nn < D / 16; ++nn) {
                uint32_t b[4];
                ldsm_x4_t(b, Vs + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * KSTR + nn * 16 + 8 * (lane >> 4));
                mma_bf16(o[2 * nn], a, b[0], b[1]);
                mma_bf16(o[2 * nn + 1], a, b[2], b[3]);
            }
        }
    }

    __device__ __forceinline__ void finish_sums() {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
            l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        }
    }
};

// ------------------------------------------------------------------ tiled kernel --
// grid.x: tiles of BM rows over all sequences (row = token*G + head in group),
// grid.y: kv heads.  Tile -> sequence by a scan of the per-sequence tile counts.
__global__ void __launch_bounds__(NTHREADS)
attn_tiled_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ cache,
                  const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_q,
                  const int* __restrict__ ctx_lens, int n_seqs, bf16* __restrict__ out, int out_stride,
                  int nq, int nkv, int block_size, int num_blocks, float scale_log2, int window,
                  int* __restrict__ status) {
    pdl_prologue();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                 // [BM][KSTR]
    bf16* Ks = Qs + BM * KSTR;                                    // [2][BN][KSTR]
    bf16* Vs = Ks + 2 * BN * KSTR;                                // [2][BN][KSTR]
    __shared__ int s_seq, s_tile;
    const int G = nq / nkv;
    const int kh = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    if (warp == 0) {   // which sequence owns tile blockIdx.x
        int base = 0, found_seq = -1, found_tile = 0;
        for (int s0 = 0; s0 < n_seqs && found_seq < 0; s0 += 32) {
            const int s = s0 + lane;
            const int cnt = s < n_seqs ? ((cu_q[s + 1] - cu_q[s]) * G + BM - 1) / BM : 0;
            int incl = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            const int total = __shfl_sync(0xffffffffu, incl, 31);
            const unsigned hit = __ballot_sync(0xffffffffu, base + incl > (int)blockIdx.x);
            if (hit) {
                const int l0 = __ffs(hit) - 1;
                found_seq = s0 + l0;
                const int incl0 = __shfl_sync(0xffffffffu, incl, l0);
                const int cnt0 = __shfl_sync(0xffffffffu, cnt, l0);
                found_tile = (int)blockIdx.x - (base + incl0 - cnt0);
            }
            base += total;
        }
        if (lane == 0) { s_seq = found_seq; s_tile = found_tile; }
    }
    __syncthreads();
    const int seq = s_seq, tile = s_tile;
    if (seq < 0) return;
    const int tok0 = cu_q[seq], q_len = cu_q[seq + 1] - tok0, ctx = ctx_lens[seq];
    const int rows = q_len * G;
    const int row0 = tile * BM;
    const int* bt = block_table + (size_t)seq * max_blocks;

    // q tile -> smem
    for (int c = threadIdx.x; c < BM * CHUNKS; c += NTHREADS) {
        const int r = c / CHUNKS, ch = c % CHUNKS;
        const int rg = row0 + r;
        const bool ok = rg < rows;
        const bf16* src = q;
        if (ok) src = q + (size_t)(tok0 + rg / G) * q_stride + (size_t)(kh * G + rg % G) * D + ch * 8;
        cp_async16(Qs + r * KSTR + ch * 8, src, ok);
    }
    // visible keys of the tile
    const int first_tok = row0 / G;
    const int last_tok = min(q_len - 1, (row0 + BM - 1) / G);
    const int kv_hi = ctx + last_tok + 1;
    const int kv_lo = window > 0 ? max(0, ctx + first_tok - window + 1) : 0;
    const int t_begin = kv_lo / BN, t_end = (kv_hi + BN - 1) / BN;

    const size_t v_off = (size_t)nkv * block_size * D;
    __shared__ long long s_row_off[2][BN];
    kv_row_offsets(s_row_off[0], bt, max_blocks, num_blocks, nkv, kh, block_size, t_begin * BN, kv_lo, kv_hi, status);
    if (t_begin + 1 < t_end)
        kv_row_offsets(s_row_off[1], bt, max_blocks, num_blocks, nkv, kh, block_size, (t_begin + 1) * BN, kv_lo, kv_hi, status);
    __syncthreads();
    load_kv_tile(Ks, Vs, cache, s_row_off[0], v_off);
    cp_async_commit();

    // this thread's two rows
    const int g = lane >> 2;
    int lo[2], hi[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int rg = row0 + warp * 16 + g + 8 * r;
        const int pos = ctx + min(rg, rows - 1) / G;
        hi[r] = pos + 1;
        lo[r] = window > 0 ? max(0, pos - window + 1) : 0;
    }
    const bool warp_active = row0 + warp * 16 < rows;
    // keys below this are visible to every row of the warp, keys at or above need the mask
    const int warp_first_pos = ctx + min(row0 + warp * 16, rows - 1) / G;
    const int warp_last_pos = ctx + min(row0 + warp * 16 + 15, rows - 1) / G;
    const int full_lo = window > 0 ? max(0, warp_last_pos - window + 1) : 0;
    const int warp_lo = window > 0 ? max(0, warp_first_pos - window + 1) : 0;   // first key any row sees

    WarpState<BN> st;
    st.init();
    for (int t = t_begin; t < t_end; ++t) {
        const int buf = (t - t_begin) & 1;
        if (t + 1 < t_end) {
            load_kv_tile(Ks + (buf ^ 1) * BN * KSTR, Vs + (buf ^ 1) * BN * KSTR, cache, s_row_off[buf ^ 1], v_off);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        // the offsets of tile t are used up: look up those of tile t+2 (read after the next barrier)
        if (t + 2 < t_end)
            kv_row_offsets(s_row_off[buf], bt, max_blocks, num_blocks, nkv, kh, block_size, (t + 2) * BN, kv_lo, kv_hi, status);
        const int key0 = t * BN;
        if (warp_active && key0 <= warp_last_pos && key0 + BN > warp_lo) {   // warp-uniform
            const bool need_mask = key0 + BN > warp_first_pos + 1 || key0 < full_lo || key0 < kv_lo;
            st.step(Qs + warp * 16 * KSTR, Ks + buf * BN * KSTR, Vs + buf * BN * KSTR, key0, lo, hi,
                    scale_log2, need_mask);
        }
        __syncthreads();
    }
    st.finish_sums();
    if (!warp_active) return;
    const int t4 = lane & 3;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int rg = row0 + warp * 16 + g + 8 * r;
        if (rg >= rows) continue;
        const float inv = 1.0f / st.l[r];
        bf16* dst = out + (size_t)(tok0 + rg / G) * out_stride + (size_t)(kh * G + rg % G) * D;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            __nv_bfloat162 v = __floats2bfloat162_rn(st.o[i][2 * r] * inv, st.o[i][2 * r + 1] * inv);
            *reinterpret_cast<__nv_bfloat162*>(dst + i * 8 + 2 * t4) = v;
        }
    }
}

// ----------------------------------------------------------------- decode kernel --
// One token per sequence.  grid (sequence, kv head, split).  The block's four warps
// share each tile of 64 keys, 16 keys a warp, and join their states at the end.
// With one split the output is final; else partial (o, m, l) go to scratch memory.
//
// HEADS = true: the kernel also finishes the heads of the newest token, which then come straight
// from the q|k|v projection (`q` is that buffer, a row being the q heads, the k heads, the v heads):
// each block normalises and rotates the query heads of its group on their way into shared memory,
// and the block whose range of keys holds the newest one does the same for that key, writes it and
// its value into the cache page and puts both into its tile.  One kernel and one pass over q|k|v
// less per layer than with the separate kernel of qk_rope_store.cu; the arithmetic is the same.
struct DecodeHeads {
    const float* q_norm_w;     // [D] or null: no per-head norm
    const float* k_norm_w;
    float eps;
    const float* cos_sin;      // [max_positions][D/2][2] or null: no rotation
    int max_positions;
    bf16* cache_w;             // the cache again, to write the newest key and value
    int* status;               // 2: page of the newest token missing, 3: position beyond the table, 4: a key's page missing
};
constexpr int HC = D / 64;     // elements of each half of a head that a lane holds (heads finished in a warp)

template <int C> __device__ __forceinline__ void load_run(bf16 (&a)[C], const bf16* p) {
    if constexpr (C % 4 == 0) {
#pragma unroll
        for (int j = 0; j < C / 4; ++j) reinterpret_cast<uint2*>(a)[j] = reinterpret_cast<const uint2*>(p)[j];
    } else if constexpr (C % 2 == 0) {
#pragma unroll
        for (int j = 0; j < C / 2; ++j) reinterpret_cast<uint32_t*>(a)[j] = reinterpret_cast<const uint32_t*>(p)[j];
    } else {
#pragma unroll
        for (int j = 0; j < C; ++j) a[j] = p[j];
    }
}
template <int C> __device__ __forceinline__ void store_run(bf16* p, const bf16 (&a)[C]) {
    if constexpr (C % 4 == 0) {
#pragma unroll
        for (int j = 0; j < C / 4; ++j) reinterpret_cast<uint2*>(p)[j] = reinterpret_cast<const uint2*>(a)[j];
    } else if constexpr (C % 2 == 0) {
#pragma unroll
        for (int j = 0; j < C / 2; ++j) reinterpret_cast<uint32_t*>(p)[j] = reinterpret_cast<const uint32_t*>(a)[j];
    } else {
#pragma unroll
        for (int j = 0; j < C; ++j) p[j] = a[j];
    }
}
// One head in a warp: lane l holds elements l*C.. of the first half (a) and their partners of the
// second half (b).  RMS norm over the head with weights (wl, wh) if `norm`, then each pair (a, b)
// turned by its angle if `rotate`; 32-bit throughout, rounded once at the end.
template <int C>
__device__ __forceinline__ void finish_head(bf16 (&a)[C], bf16 (&b)[C], bool norm, const float (&wl)[C],
                                            const float (&wh)[C], float eps, bool rotate,
                                            const float (&cs_c)[C], const float (&cs_s)[C]) {
    float lo[C], hi[C];
#pragma unroll
    for (int j = 0; j < C; ++j) { lo[j] = __bfloat162float(a[j]); hi[j] = __bfloat162float(b[j]); }
    if (norm) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < C; ++j) ss += lo[j] * lo[j] + hi[j] * hi[j];
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)(64 * C) + eps);
#pragma unroll
        for (int j = 0; j < C; ++j) {
            lo[j] = lo[j] * inv * wl[j];
            hi[j] = hi[j] * inv * wh[j];
        }
    }
    if (rotate) {
#pragma unroll
        for (int j = 0; j < C; ++j) {
            const float x = lo[j], y = hi[j];
            lo[j] = x * cs_c[j] - y * cs_s[j];
            hi[j] = y * cs_c[j] + x * cs_s[j];
        }
    }
#pragma unroll
    for (int j = 0; j < C; ++j) { a[j] = __float2bfloat16_rn(lo[j]); b[j] = __float2bfloat16_rn(hi[j]); }
}

// UNITS = true: the ranges of keys are given out by length.  grid (kv head, unit): the units are
// shared out among the sequences in proportion to their tiles of keys, one at least for each, so
// that a step's blocks fill the SMs' places exactly once whatever the lengths are (a fixed number
// of ranges per sequence leaves places empty or starts a second round).  Every block works the
// share-out out for itself from the context lengths, before it waits for the kernel in front.
struct DecodeUnits {
    int n_seqs;                // at most NTHREADS, at most gridDim.y
    int max_ranges;            // no sequence is cut into more ranges than this
    int* seq_ranges;           // [n_seqs] out: the number of ranges of each sequence, for the join
    int part_stride;           // partial results of a (sequence, head) lie this many apart
};

template <bool HEADS, bool UNITS>
__device__ __forceinline__ void
attn_decode_body(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ cache,
                 const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_q,
                 const int* __restrict__ ctx_lens, bf16* __restrict__ out, int out_stride,
                 float* __restrict__ part_o, float* __restrict__ part_ml, int nq, int nkv,
                 int block_size, int num_blocks, float scale_log2, int window, int num_splits,
                 const DecodeHeads& hd, const DecodeUnits& un) {
    // The kernel in front of this one (per-head norm, rotation and cache write, or the projection
    // itself) produces q and the newest key and value only.  The step's metadata and every older key
    // do not depend on it: they are fetched before the wait for that kernel, so the first tile is
    // on its way when it ends.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                 // [16][KSTR]
    bf16* Ks = Qs + 16 * KSTR;                                    // [2][BN][KSTR]
    bf16* Vs = Ks + 2 * BN * KSTR;                                // [2][BN][KSTR]
    const int G = nq / nkv;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int seq, kh, split, ranges, part_stride, pos;
    if constexpr (UNITS) {
        __shared__ int s_warp_tiles[NTHREADS / 32];
        __shared__ int s_mine[4];
        kh = blockIdx.x;
        const int unit = blockIdx.y, units = gridDim.y, n = un.n_seqs;
        const int i = threadIdx.x;                                 // thread i looks at sequence i
        int tiles = 0, p = 0;
        if (i < n) {
            p = ctx_lens[i];
            tiles = (p + BN) / BN - (window > 0 ? max(0, p - window + 1) : 0) / BN;
        }
        int incl = tiles;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) s_warp_tiles[warp] = incl;
        if (i == 0) s_mine[0] = -1;
        __syncthreads();
        int before = 0, all = 0;
#pragma unroll
        for (int w = 0; w < NTHREADS / 32; ++w) {
            if (w < warp) before += s_warp_tiles[w];
            all += s_warp_tiles[w];
        }
        // sequence i owns the units [i + spare * tiles before it / all, i + 1 + spare * tiles up to it / all);
        // the host has seen to it that spare * all fits 31 bits
        const unsigned spare = units - n;
        const unsigned excl = before + incl - tiles;
        const int u0 = i + (int)(spare * excl / (unsigned)all);
        const int u1 = i + 1 + (int)(spare * (excl + tiles) / (unsigned)all);
        if (i < n && unit >= u0 && unit < u1) {
            s_mine[0] = i;
            s_mine[1] = unit - u0;
            // a range holds a tile and a half of keys at least: short sequences are not cut into crumbs
            s_mine[2] = min(min(u1 - u0, max(1, tiles * 2 / 3)), un.max_ranges);
            s_mine[3] = p;
        }
        __syncthreads();
        seq = s_mine[0];
        split = s_mine[1];
        ranges = s_mine[2];
        part_stride = un.part_stride;
        if (seq < 0 || split >= ranges) return;                    // a unit without work
        pos = s_mine[3];
    } else {
        seq = blockIdx.x;
        kh = blockIdx.y;
        split = blockIdx.z;
        ranges = num_splits;
        part_stride = num_splits;
        pos = ctx_lens[seq];
    }
    const int tok = cu_q[seq];
    const int kv_hi = pos + 1;
    const int kv_lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* bt = block_table + (size_t)seq * max_blocks;
    const int t0 = kv_lo / BN, t1 = (kv_hi + BN - 1) / BN;
    int t_begin, t_end;
    if constexpr (UNITS) {       // ranges <= tiles: none is empty, and they differ by one tile at most
        t_begin = t0 + (unsigned)((t1 - t0) * split) / (unsigned)ranges;
        t_end = t0 + (unsigned)((t1 - t0) * (split + 1)) / (unsigned)ranges;
    } else {
        const int per = (t1 - t0 + ranges - 1) / ranges;
        t_begin = t0 + split * per;
        t_end = min(t1, t_begin + per);
    }

    const size_t v_off = (size_t)nkv * block_size * D;
    __shared__ long long s_row_off[2][BN];
    if (t_begin < t_end)
        kv_row_offsets(s_row_off[0], bt, max_blocks, num_blocks, nkv, kh, block_size, t_begin * BN, kv_lo, kv_hi, hd.status);
    if (t_begin + 1 < t_end)
        kv_row_offsets(s_row_off[1], bt, max_blocks, num_blocks, nkv, kh, block_size, (t_begin + 1) * BN, kv_lo, kv_hi, hd.status);
    __syncthreads();
    // the first tile can go early if it ends before the newest key, or if that key is put into the tile later
    const bool early = t_begin < t_end && (HEADS || (t_begin + 1) * BN <= pos);
    if (early) load_kv_tile(Ks, Vs, cache, s_row_off[0], v_off);
    if constexpr (HEADS) {           // no key in the pages depends on the kernel in front: the second tile goes too
        cp_async_commit();
        if (t_begin + 1 < t_end) load_kv_tile(Ks + BN * KSTR, Vs + BN * KSTR, cache, s_row_off[1], v_off);
        cp_async_commit();
    }
    // HEADS: what the finishing of the heads needs besides the projection's output
    constexpr int C = HC > 0 ? HC : 1;
    const int t_last = pos / BN;                                  // the tile of the newest key
    const bool owner = HEADS && t_begin <= t_last && t_last < t_end;
    const int e0 = lane * C;
    float wl[C], wh[C], cs_c[C], cs_s[C];
    __align__(8) bf16 new_a[C], new_b[C];                         // warp 0: the newest key, warp 1: its value
    bool rotate = false, pos_ok = true;
    int new_page = -1;
    if constexpr (HEADS) {
        rotate = hd.cos_sin != nullptr;
        pos_ok = pos >= 0 && pos < hd.max_positions;
#pragma unroll
        for (int j = 0; j < C; ++j) {
            wl[j] = hd.q_norm_w ? hd.q_norm_w[e0 + j] : 1.f;
            wh[j] = hd.q_norm_w ? hd.q_norm_w[D / 2 + e0 + j] : 1.f;
            cs_c[j] = 1.f;
            cs_s[j] = 0.f;
            if (rotate && pos_ok) {
                const float* cs = hd.cos_sin + (size_t)pos * D + 2 * (e0 + j);
                cs_c[j] = cs[0];
                cs_s[j] = cs[1];
            }
        }
        if (owner && warp < 2) new_page = (pos >= 0 && pos / block_size < max_blocks) ? bt[pos / block_size] : -1;
        // rows of the tile beyond the group are zeros
        for (int c = G * CHUNKS + threadIdx.x; c < 16 * CHUNKS; c += NTHREADS)
            *reinterpret_cast<uint4*>(Qs + (c / CHUNKS) * KSTR + (c % CHUNKS) * 8) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if constexpr (UNITS) {
        if (split == 0 && kh == 0 && threadIdx.x == 0) un.seq_ranges[seq] = ranges;
    }
    if constexpr (HEADS) {
        const bf16* row = q + (size_t)tok * q_stride;
        if (owner && warp < 2) {
            // the newest key (warp 0) and value (warp 1) are asked for beside the query heads
            const bf16* src = row + (size_t)(nq + warp * nkv + kh) * D;
            load_run<C>(new_a, src + e0);
            load_run<C>(new_b, src + D / 2 + e0);
        }
        for (int r = warp; r < G; r += NTHREADS / 32) {
            __align__(8) bf16 a[C], b[C];
            const bf16* src = row + (size_t)(kh * G + r) * D;
            load_run<C>(a, src + e0);
            load_run<C>(b, src + D / 2 + e0);
            finish_head<C>(a, b, hd.q_norm_w != nullptr, wl, wh, hd.eps, rotate && pos_ok, cs_c, cs_s);
            store_run<C>(Qs + r * KSTR + e0, a);
            store_run<C>(Qs + r * KSTR + D / 2 + e0, b);
        }
        if (rotate && !pos_ok && threadIdx.x == 0) atomicExch(hd.status, 3);
        if (owner && warp < 2) {
            if (warp == 0) {
                float kl[C], kh_w[C];
#pragma unroll
                for (int j = 0; j < C; ++j) {
                    kl[j] = hd.k_norm_w ? hd.k_norm_w[e0 + j] : 1.f;
                    kh_w[j] = hd.k_norm_w ? hd.k_norm_w[D / 2 + e0 + j] : 1.f;
                }
                finish_head<C>(new_a, new_b, hd.k_norm_w != nullptr, kl, kh_w, hd.eps, rotate && pos_ok, cs_c, cs_s);
            }
            if (new_page >= 0 && new_page < num_blocks) {
                bf16* dst = hd.cache_w +
                            ((((size_t)new_page * 2 + warp) * nkv + kh) * block_size + pos % block_size) * D;
                store_run<C>(dst + e0, new_a);
                store_run<C>(dst + D / 2 + e0, new_b);
            } else if (lane == 0) {
                atomicExch(hd.status, 2);
            }
        }
    } else {
        for (int c = threadIdx.x; c < 16 * CHUNKS; c += NTHREADS) {
            const int r = c / CHUNKS, ch = c % CHUNKS;
            const bool ok = r < G;
            const bf16* src = ok ? q + (size_t)tok * q_stride + (size_t)(kh * G + r) * D + ch * 8 : q;
            cp_async16(Qs + r * KSTR + ch * 8, src, ok);
        }
    }
    if constexpr (!HEADS) {
        if (!early && t_begin < t_end) load_kv_tile(Ks, Vs, cache, s_row_off[0], v_off);
        cp_async_commit();
        if (t_begin + 1 < t_end) load_kv_tile(Ks + BN * KSTR, Vs + BN * KSTR, cache, s_row_off[1], v_off);
        cp_async_commit();
    }

    int lo[2] = {kv_lo, kv_lo}, hi[2] = {kv_hi, kv_hi};
    WarpState<16> st;
    st.init();
    for (int t = t_begin; t < t_end; ++t) {
        const int buf = (t - t_begin) & 1;
        if (t + 1 < t_end) {
            if (t != t_begin) {      // the first two tiles were asked for above
                load_kv_tile(Ks + (buf ^ 1) * BN * KSTR, Vs + (buf ^ 1) * BN * KSTR, cache, s_row_off[buf ^ 1], v_off);
                cp_async_commit();
            }
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (HEADS && owner && t == t_last) {
            // the tile's copy of the newest row may be older than this block's write to the page:
            // the finished key and value go into the tile from the registers that hold them
            if (warp < 2) {
                bf16* dst = (warp == 0 ? Ks : Vs) + (buf * BN + (pos - t_last * BN)) * KSTR;
                store_run<C>(dst + e0, new_a);
                store_run<C>(dst + D / 2 + e0, new_b);
            }
            __syncthreads();
        }
        // the offsets of tile t are used up: look up those of tile t+2.  The page id is asked for now and
        // written to shared memory after this tile's arithmetic, so its trip to memory costs nothing.
        const bool look = t + 2 < t_end && threadIdx.x < BN;
        long long off_next = -1;
        if (look)
            off_next = kv_row_offset(bt, max_blocks, num_blocks, nkv, kh, block_size, (t + 2) * BN + threadIdx.x, kv_lo, kv_hi, hd.status);
        const int key0 = t * BN + warp * 16;
        if (key0 < kv_hi && key0 + 16 > kv_lo) {
            const bool need_mask = key0 + 16 > kv_hi || key0 < kv_lo;
            st.step(Qs, Ks + (buf * BN + warp * 16) * KSTR, Vs + (buf * BN + warp * 16) * KSTR, key0, lo, hi,
                    scale_log2, need_mask);
        }
        if (look) s_row_off[buf][threadIdx.x] = off_next;
        __syncthreads();
    }
    cp_async_wait<0>();
    st.finish_sums();
    __syncthreads();
    // join the four warps: rows g and g+8 of each, of which only the group's rows (< G) are kept.
    // A row is D + 8 floats apart from the next, so the quads of a warp store to distinct banks.
    constexpr int JSTR = D + 8;
    float* sm_o = reinterpret_cast<float*>(Ks);                   // [4][16][JSTR]
    float* sm_m = sm_o + 4 * 16 * JSTR;                           // [4][16]
    float* sm_l = sm_m + 4 * 16;                                  // [4][16]
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = g + 8 * r;
        if (row >= G) continue;
        if (t4 == 0) { sm_m[warp * 16 + row] = st.m[r]; sm_l[warp * 16 + row] = st.l[r]; }
#pragma unroll
        for (int i = 0; i < D / 8; ++i)
            *reinterpret_cast<float2*>(sm_o + (warp * 16 + row) * JSTR + i * 8 + 2 * t4) =
                make_float2(st.o[i][2 * r], st.o[i][2 * r + 1]);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += NTHREADS) {
        const int row = idx / D, col = idx % D;
        float M = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w * 16 + row]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = sm_m[w * 16 + row];
            const float wt = mw == -CUDART_INF_F ? 0.f : exp2f(mw - M);
            L += wt * sm_l[w * 16 + row];
            O += wt * sm_o[(w * 16 + row) * JSTR + col];
        }
        const int head = kh * G + row;
        if (ranges == 1) {
            out[(size_t)tok * out_stride + (size_t)head * D + col] = __float2bfloat16_rn(O / L);
        } else {
            const size_t p = ((size_t)seq * nq + head) * part_stride + split;
            part_o[p * D + col] = O;
            if (col == 0) { part_ml[p * 2] = M; part_ml[p * 2 + 1] = L; }
        }
    }
}

__global__ void __launch_bounds__(NTHREADS)
attn_decode_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ cache,
                   const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_q,
                   const int* __restrict__ ctx_lens, bf16* __restrict__ out, int out_stride,
                   float* __restrict__ part_o, float* __restrict__ part_ml, int nq, int nkv,
                   int block_size, int num_blocks, float scale_log2, int window, int num_splits,
                   int* __restrict__ status) {
    DecodeHeads hd{};
    hd.status = status;           // may be null: a missing page is then not reported
    attn_decode_body<false, false>(q, q_stride, cache, block_table, max_blocks, cu_q, ctx_lens, out, out_stride,
                                   part_o, part_ml, nq, nkv, block_size, num_blocks, scale_log2, window, num_splits,
                                   hd, DecodeUnits{});
}
__global__ void __launch_bounds__(NTHREADS)
attn_decode_heads_kernel(const bf16* __restrict__ qkv, int row_width, const bf16* __restrict__ cache,
                         const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_q,
                         const int* __restrict__ ctx_lens, bf16* __restrict__ out, int out_stride,
                         float* __restrict__ part_o, float* __restrict__ part_ml, int nq, int nkv,
                         int block_size, int num_blocks, float scale_log2, int window, int num_splits,
                         DecodeHeads hd) {
    if constexpr (D % 64 == 0)
        attn_decode_body<true, false>(qkv, row_width, cache, block_table, max_blocks, cu_q, ctx_lens, out,
                                      out_stride, part_o, part_ml, nq, nkv, block_size, num_blocks, scale_log2,
                                      window, num_splits, hd, DecodeUnits{});
}
// grid (kv head, unit); HEADS as above
template <bool HEADS>
__global__ void __launch_bounds__(NTHREADS)
attn_decode_units_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ cache,
                         const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_q,
                         const int* __restrict__ ctx_lens, bf16* __restrict__ out, int out_stride,
                         float* __restrict__ part_o, float* __restrict__ part_ml, int nq, int nkv,
                         int block_size, int num_blocks, float scale_log2, int window, DecodeHeads hd,
                         DecodeUnits un) {
    if constexpr (!HEADS || D % 64 == 0)
        attn_decode_body<HEADS, true>(q, q_stride, cache, block_table, max_blocks, cu_q, ctx_lens, out, out_stride,
                                      part_o, part_ml, nq, nkv, block_size, num_blocks, scale_log2, window, 0, hd,
                                      un);
}

// out[token of seq, head, :] = sum_s w_s o_s / sum_s w_s l_s,  w_s = 2^(m_s - max m).
// The splits are taken eight at a time, all their loads issued before the first is used (one
// trip to memory for up to eight splits), with a running maximum over the groups of eight.
// seq_ranges given: sequence s has seq_ranges[s] partial results, part_stride apart per (sequence,
// head); with one range its output is final already.
__device__ __forceinline__ void attn_combine_body(const float* __restrict__ part_o,
                                                  const float* __restrict__ part_ml,
                                                  const int* __restrict__ cu_q, bf16* __restrict__ out,
                                                  int out_stride, int nq, int num_splits,
                                                  const int* __restrict__ seq_ranges, int part_stride) {
    pdl_prologue();
    const int seq = blockIdx.x, head = blockIdx.y;
    // The count of a sequence's partial results is asked for together with the first eight of them
    // (which may lie beyond the count: they are read from the scratch memory and then ignored).
    const int readable = seq_ranges != nullptr ? part_stride : num_splits;
    if (seq_ranges != nullptr) num_splits = seq_ranges[seq];
    const size_t base = ((size_t)seq * nq + head) * part_stride;
    const int tok = cu_q[seq];
    for (int col = threadIdx.x; col < D; col += blockDim.x) {
        float M = -CUDART_INF_F, L = 0.f, O = 0.f;
        for (int s0 = 0; s0 == 0 || s0 < num_splits; s0 += 8) {
            float ms[8], ls[8], os[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const size_t p = base + min(s0 + k, readable - 1);
                ms[k] = part_ml[p * 2];
                ls[k] = part_ml[p * 2 + 1];
                os[k] = part_o[p * D + col];
            }
            if (seq_ranges != nullptr && num_splits <= 1) return;   // one range: the output is final already
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (s0 + k >= num_splits) ms[k] = -CUDART_INF_F;
            float Mn = M;
#pragma unroll
            for (int k = 0; k < 8; ++k) Mn = fmaxf(Mn, ms[k]);
            if (Mn == -CUDART_INF_F) continue;                     // no key in any split so far
            const float r = M == -CUDART_INF_F ? 0.f : exp2f(M - Mn);
            L *= r;
            O *= r;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (ms[k] != -CUDART_INF_F) {
                    const float w = exp2f(ms[k] - Mn);
                    L += w * ls[k];
                    O += w * os[k];
                }
            }
            M = Mn;
        }
        out[(size_t)tok * out_stride + (size_t)head * D + col] = __float2bfloat16_rn(O / L);
    }
}
__device__ __forceinline__ void attn_combine_many_body(const float* __restrict__ part_o,
                                                  const float* __restrict__ part_ml,
                                                  const int* __restrict__ cu_q, bf16* __restrict__ out,
                                                  int out_stride, int nq, int num_splits,
                                                  const int* __restrict__ seq_ranges, int part_stride) {
    pdl_prologue();
    // The form for many ranges (a long sequence cut into up to 64).  It holds shared memory, so its blocks
    // cannot sit beside three blocks of the attention kernel and start only when those leave: the form
    // above, which holds none, stays the one for the usual few ranges (0.9 us a layer at batch 8).
    // D / 4 threads (four columns each, 16-byte loads) make a group; the block's groups take the
    // partial results in turn (group g the ranges g, g + groups, ...), four loads in flight each, and
    // group 0 then merges the groups' sums in their order: the result does not depend on timing.
    constexpr int LPG = D / 4;
    constexpr int MAXG = 8;
    __shared__ float s_o[MAXG][D];
    __shared__ float s_ml[MAXG][2];
    const int seq = blockIdx.x, head = blockIdx.y;
    const int groups = min(MAXG, (int)blockDim.x / LPG);
    const int g = threadIdx.x / LPG, col = (threadIdx.x % LPG) * 4;
    if (seq_ranges != nullptr) num_splits = seq_ranges[seq];
    if (seq_ranges != nullptr && num_splits <= 1) return;          // one range: the output is final already
    const size_t base = ((size_t)seq * nq + head) * part_stride;
    const int tok = cu_q[seq];
    float M = -CUDART_INF_F, L = 0.f;
    float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
    if (g < groups) {
        for (int s0 = g; s0 < num_splits; s0 += 4 * groups) {
            float ms[4], ls[4];
            float4 os[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int sp = s0 + k * groups;
                const size_t p = base + min(sp, num_splits - 1);
                const float2 ml = *reinterpret_cast<const float2*>(part_ml + p * 2);
                ms[k] = sp < num_splits ? ml.x : -CUDART_INF_F;
                ls[k] = ml.y;
                os[k] = *reinterpret_cast<const float4*>(part_o + p * D + col);
            }
            float Mn = M;
#pragma unroll
            for (int k = 0; k < 4; ++k) Mn = fmaxf(Mn, ms[k]);
            if (Mn == -CUDART_INF_F) continue;                     // no key in any of these ranges
            const float r = M == -CUDART_INF_F ? 0.f : exp2f(M - Mn);
            L *= r;
            O.x *= r; O.y *= r; O.z *= r; O.w *= r;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (ms[k] != -CUDART_INF_F) {
                    const float w = exp2f(ms[k] - Mn);
                    L += w * ls[k];
                    O.x += w * os[k].x; O.y += w * os[k].y; O.z += w * os[k].z; O.w += w * os[k].w;
                }
            }
            M = Mn;
        }
        *reinterpret_cast<float4*>(&s_o[g][col]) = O;
        if (col == 0) { s_ml[g][0] = M; s_ml[g][1] = L; }
    }
    __syncthreads();
    if (g == 0) {
        float Mt = -CUDART_INF_F;
        for (int k = 0; k < groups; ++k) Mt = fmaxf(Mt, s_ml[k][0]);
        float Lt = 0.f;
        float4 Ot = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < groups; ++k) {
            const float mk = s_ml[k][0];
            if (mk == -CUDART_INF_F) continue;
            const float w = exp2f(mk - Mt);
            const float4 o = *reinterpret_cast<const float4*>(&s_o[k][col]);
            Lt += w * s_ml[k][1];
            Ot.x += w * o.x; Ot.y += w * o.y; Ot.z += w * o.z; Ot.w += w * o.w;
        }
        const float inv = 1.0f / Lt;
        __align__(8) bf16 r4[4] = {__float2bfloat16_rn(Ot.x * inv), __float2bfloat16_rn(Ot.y * inv),
                                   __float2bfloat16_rn(Ot.z * inv), __float2bfloat16_rn(Ot.w * inv)};
        *reinterpret_cast<uint2*>(out + (size_t)tok * out_stride + (size_t)head * D + col) = *reinterpret_cast<const uint2*>(r4);
    }
}
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    const int* __restrict__ cu_q, bf16* __restrict__ out, int out_stride,
                                    int nq, int num_splits) {
    attn_combine_body(part_o, part_ml, cu_q, out, out_stride, nq, num_splits, nullptr, num_splits);
}
__global__ void attn_combine_units_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                          const int* __restrict__ cu_q, bf16* __restrict__ out, int out_stride,
                                          int nq, const int* __restrict__ seq_ranges, int part_stride) {
    attn_combine_body(part_o, part_ml, cu_q, out, out_stride, nq, 0, seq_ranges, part_stride);
}
__global__ void attn_combine_many_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         const int* __restrict__ cu_q, bf16* __restrict__ out, int out_stride,
                                         int nq, int num_splits) {
    attn_combine_many_body(part_o, part_ml, cu_q, out, out_stride, nq, num_splits, nullptr, num_splits);
}
__global__ void attn_combine_units_many_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                               const int* __restrict__ cu_q, bf16* __restrict__ out, int out_stride,
                                               int nq, const int* __restrict__ seq_ranges, int part_stride) {
    attn_combine_many_body(part_o, part_ml, cu_q, out, out_stride, nq, 0, seq_ranges, part_stride);
}

constexpr int COMBINE_THREADS = D >= 256 ? 256 : 128;     // two to eight groups of D / 4 threads
constexpr size_t TILED_SMEM = (size_t)(BM + 4 * BN) * KSTR * sizeof(bf16);
constexpr size_t DECODE_KV_SMEM = (size_t)(4 * BN) * KSTR * sizeof(bf16);
constexpr size_t DECODE_JOIN_SMEM = (size_t)(4 * 16 * (D + 8) + 2 * 4 * 16) * sizeof(float);
constexpr size_t DECODE_SMEM = (size_t)16 * KSTR * sizeof(bf16) +
                               (DECODE_KV_SMEM > DECODE_JOIN_SMEM ? DECODE_KV_SMEM : DECODE_JOIN_SMEM);

}  // namespace ff

using namespace ff;

FF_EXPORT int ff_attn_head_dim() { return D; }
FF_EXPORT int ff_attn_block_m() { return BM; }

// total_tiles = sum over sequences of ceil(q_len * G / BM)
FF_EXPORT int ff_attn_tiled(const void* q, int q_stride, const void* cache, const int* block_table,
                            int max_blocks, const int* cu_q, const int* ctx_lens, int n_seqs,
                            int total_tiles, void* out, int out_stride, int nq, int nkv, int block_size,
                            int num_blocks, float scale, int window, int* status, cudaStream_t stream) {
    if (n_seqs <= 0 || total_tiles <= 0) return 0;
    if (nkv <= 0 || nq % nkv) return FF_ERR_BAD_ARG;
    FF_SMEM_LIMIT(attn_tiled_kernel, TILED_SMEM);
    dim3 grid(total_tiles, nkv);
    FF_LAUNCH((attn_tiled_kernel), grid, NTHREADS, TILED_SMEM, stream, 
        (const bf16*)q, q_stride, (const bf16*)cache, block_table, max_blocks, cu_q, ctx_lens, n_seqs,
        (bf16*)out, out_stride, nq, nkv, block_size, num_blocks, scale * LOG2E, window, status);
    FF_LAUNCH_CHECK();
    return 0;
}

// Every sequence has exactly one token.  part_o: float [n_seqs*nq*num_splits*D],
// part_ml: float [n_seqs*nq*num_splits*2] (unused when num_splits == 1).
FF_EXPORT int ff_attn_decode(const void* q, int q_stride, const void* cache, const int* block_table,
                             int max_blocks, const int* cu_q, const int* ctx_lens, int n_seqs, void* out,
                             int out_stride, float* part_o, float* part_ml, int nq, int nkv,
                             int block_size, int num_blocks, float scale, int window, int num_splits,
                             int* status, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (nkv <= 0 || nq % nkv || num_splits < 1) return FF_ERR_BAD_ARG;
    if (nq / nkv > 16) return FF_ERR_UNSUPPORTED;
    FF_SMEM_LIMIT(attn_decode_kernel, DECODE_SMEM);
    dim3 grid(n_seqs, nkv, num_splits);
    FF_LAUNCH((attn_decode_kernel), grid, NTHREADS, DECODE_SMEM, stream, 
        (const bf16*)q, q_stride, (const bf16*)cache, block_table, max_blocks, cu_q, ctx_lens, (bf16*)out,
        out_stride, part_o, part_ml, nq, nkv, block_size, num_blocks, scale * LOG2E, window, num_splits, status);
    FF_LAUNCH_CHECK();
    if (num_splits > 1) {
        dim3 cgrid(n_seqs, nq);
        if (num_splits > 8)
            FF_LAUNCH((attn_combine_many_kernel), cgrid, COMBINE_THREADS, 0, stream, part_o, part_ml, cu_q, (bf16*)out,
                      out_stride, nq, num_splits);
        else
            FF_LAUNCH((attn_combine_kernel), cgrid, D >= 128 ? 128 : 64, 0, stream, part_o, part_ml, cu_q, (bf16*)out,
                      out_stride, nq, num_splits);
        FF_LAUNCH_CHECK();
    }
    return 0;
}

// The same with the heads of the newest token finished inside the kernel: `qkv` is the raw output
// of the q|k|v projection ([tokens][row_width]: q heads, k heads, v heads), the norm weights may be
// null (no per-head norm), cos_sin may be null (no rotation; else the whole head is rotated).
// Head sizes that are multiples of 64 only.
FF_EXPORT int ff_attn_decode_heads(const void* qkv, int row_width, void* cache, const int* block_table,
                                   int max_blocks, const int* cu_q, const int* ctx_lens, int n_seqs, void* out,
                                   int out_stride, float* part_o, float* part_ml, int nq, int nkv,
                                   int block_size, int num_blocks, float scale, int window, int num_splits,
                                   const float* q_norm_w, const float* k_norm_w, float eps,
                                   const float* cos_sin, int max_positions, int* status, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (nkv <= 0 || nq % nkv || num_splits < 1 || status == nullptr) return FF_ERR_BAD_ARG;
    if (nq / nkv > 16 || D % 64 != 0) return FF_ERR_UNSUPPORTED;
    FF_SMEM_LIMIT(attn_decode_heads_kernel, DECODE_SMEM);
    DecodeHeads hd{q_norm_w, k_norm_w, eps, cos_sin, max_positions, (bf16*)cache, status};
    dim3 grid(n_seqs, nkv, num_splits);
    FF_LAUNCH((attn_decode_heads_kernel), grid, NTHREADS, DECODE_SMEM, stream,
        (const bf16*)qkv, row_width, (const bf16*)cache, block_table, max_blocks, cu_q, ctx_lens, (bf16*)out,
        out_stride, part_o, part_ml, nq, nkv, block_size, num_blocks, scale * LOG2E, window, num_splits, hd);
    FF_LAUNCH_CHECK();
    if (num_splits > 1) {
        dim3 cgrid(n_seqs, nq);
        if (num_splits > 8)
            FF_LAUNCH((attn_combine_many_kernel), cgrid, COMBINE_THREADS, 0, stream, part_o, part_ml, cu_q, (bf16*)out,
                      out_stride, nq, num_splits);
        else
            FF_LAUNCH((attn_combine_kernel), cgrid, D >= 128 ? 128 : 64, 0, stream, part_o, part_ml, cu_q, (bf16*)out,
                      out_stride, nq, num_splits);
        FF_LAUNCH_CHECK();
    }
    return 0;
}

// The ranges of keys shared out by length (see DecodeUnits): `units` blocks per kv head, of which
// every sequence gets one at least (n_seqs <= units, n_seqs <= 128).  part_o: float
// [n_seqs*nq*units*D], part_ml: float [n_seqs*nq*units*2], seq_ranges: int [n_seqs].
// finish_heads != 0: `q` is the raw q|k|v projection and the arguments behind it are used as in
// ff_attn_decode_heads; else they are ignored and q holds finished heads.
FF_EXPORT int ff_attn_decode_units(const void* q, int q_stride, void* cache, const int* block_table,
                                   int max_blocks, const int* cu_q, const int* ctx_lens, int n_seqs, void* out,
                                   int out_stride, float* part_o, float* part_ml, int* seq_ranges, int nq,
                                   int nkv, int block_size, int num_blocks, float scale, int window, int units,
                                   int max_ranges, int finish_heads, const float* q_norm_w,
                                   const float* k_norm_w, float eps, const float* cos_sin, int max_positions,
                                   int* status, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (nkv <= 0 || nq % nkv || units < n_seqs || n_seqs > NTHREADS || max_ranges < 1 || seq_ranges == nullptr)
        return FF_ERR_BAD_ARG;
    // the share-out multiplies (units - n_seqs) by a count of tiles: both within 31 bits together
    const long long most_tiles = ((long long)max_blocks * block_size / BN + 2) * n_seqs;
    if (most_tiles * (units - n_seqs + max_ranges) >= (1ll << 31)) return FF_ERR_UNSUPPORTED;
    if (nq / nkv > 16) return FF_ERR_UNSUPPORTED;
    if (finish_heads && (D % 64 != 0 || status == nullptr)) return FF_ERR_UNSUPPORTED;
    FF_SMEM_LIMIT(attn_decode_units_kernel<true>, DECODE_SMEM);
    FF_SMEM_LIMIT(attn_decode_units_kernel<false>, DECODE_SMEM);
    DecodeHeads hd{q_norm_w, k_norm_w, eps, cos_sin, max_positions, (bf16*)cache, status};
    DecodeUnits un{n_seqs, max_ranges, seq_ranges, units};
    dim3 grid(nkv, units);
    if (finish_heads)
        FF_LAUNCH((attn_decode_units_kernel<true>), grid, NTHREADS, DECODE_SMEM, stream,
            (const bf16*)q, q_stride, (const bf16*)cache, block_table, max_blocks, cu_q, ctx_lens, (bf16*)out,
            out_stride, part_o, part_ml, nq, nkv, block_size, num_blocks, scale * LOG2E, window, hd, un);
    else
        FF_LAUNCH((attn_decode_units_kernel<false>), grid, NTHREADS, DECODE_SMEM, stream,
            (const bf16*)q, q_stride, (const bf16*)cache, block_table, max_blocks, cu_q, ctx_lens, (bf16*)out,
            out_stride, part_o, part_ml, nq, nkv, block_size, num_blocks, scale * LOG2E, window, hd, un);
    FF_LAUNCH_CHECK();
    if (units > n_seqs && max_ranges > 1) {
        dim3 cgrid(n_seqs, nq);
        // a sequence gets at most this many ranges: many of them take the form that spreads them over warps
        const int most = max_ranges < units - n_seqs + 1 ? max_ranges : units - n_seqs + 1;
        if (most > 8)
            FF_LAUNCH((attn_combine_units_many_kernel), cgrid, COMBINE_THREADS, 0, stream, part_o, part_ml, cu_q,
                      (bf16*)out, out_stride, nq, (const int*)seq_ranges, units);
        else
            FF_LAUNCH((attn_combine_units_kernel), cgrid, D >= 128 ? 128 : 64, 0, stream, part_o, part_ml, cu_q,
                      (bf16*)out, out_stride, nq, (const int*)seq_ranges, units);
        FF_LAUNCH_CHECK();
    }
    return 0;
}

// Blocks of the decode kernel that one SM holds at a time (shared memory and registers).
FF_EXPORT int ff_attn_decode_blocks_per_sm() {
    // an SM has 228 KB for its blocks, each taking 1 KB besides what it asks for; 64 K registers at up to 128 a thread
    const int by_smem = (int)((228 * 1024) / (DECODE_SMEM + 1024 + 1088));
    const int by_regs = 65536 / (128 * NTHREADS);
    return by_smem < 1 ? 1 : (by_smem > by_regs ? by_regs : by_smem);
}
