// Flash-style attention over the paged cache on the fifth-generation tensor cores, for
// portions of prompts (and any mix of sequences) in bfloat16.
//
// A block owns 128 rows of one kv head (row = token * G + head-in-group, so the heads of a
// group share every key and value it fetches) and walks the visible keys in tiles of 64:
//   S = Q K^T      tcgen05.mma, Q and K from shared memory (K brought in by TMA, page by page),
//                  S (128 x 64, float32) in tensor memory;
//                  S (128 x 64, float32) in tensor memory, two buffers, so that the product for
//                  the next tile runs while the softmax works on this one;
//   softmax        four warps, one thread per row: tcgen05.ld of its row of S, mask, running max
//                  and sum in 32-bit, P as bfloat16 written back over S in tensor memory
//                  (tcgen05.st), and - only when a row's max moved far - a rescale of its row of O;
//   O += P V       tcgen05.mma, P from tensor memory, V (the cache's [key][d] tile as it is, the
//                  MMA's N-major operand form), O (128 x D, float32) in tensor memory.
// One warp starts the TMA copies, a page and panel per lane (K and V have two stages each, freed
// separately); one warp issues the MMAs, converged, with the issuing lane predicated; two blocks
// share an SM (at head size 128).
//
// It replaces, for head sizes that are multiples of 64 and page sizes that divide 64, the
// mma.sync kernel of attention_mma.cu (which stays for every other size); the reference's
// prefill kernel is a WMMA kernel over the portion's own k and v (src/kernels/attention.cu:22-286).
// Every mbarrier wait is bounded; on time-out the kernel records code 107 in the status word,
// stops, frees its tensor memory and returns.
//
// Compiled once per head size: -DFF_HEAD_DIM=<64, 128, 192 or 256>.
// Cache layout of a slot: [num_blocks][2 (k,v)][n_kv_heads][block_size][head_dim].
#include "common.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>
#include <math_constants.h>

#include <cstring>
#include <mutex>
#include <unordered_map>

#ifndef FF_HEAD_DIM
#define FF_HEAD_DIM 128
#endif

namespace ff {

constexpr int D = FF_HEAD_DIM;
static_assert(D % 64 == 0 && D >= 64 && D <= 256, "head size must be 64, 128, 192 or 256");
constexpr int BM = 128;                 // rows per block (MMA M)
constexpr int BN = 64;                  // keys per tile
constexpr int PANELS = D / 64;          // 64-column (128-byte) panels of a row
constexpr int KV_STAGES = 2;
constexpr int ATC_THREADS = 192;        // warps 0-3 softmax, warp 4 loads, warp 5 MMAs
// Page ids of a block's tiles kept in shared memory: a ring of two halves.  The softmax warps fill
// what the first tiles need; the load warp refills a half whenever its tiles move into it, so a
// context of any length is walked through the same few kilobytes.  (A test build makes it tiny.)
#ifndef FF_ATC_PAGE_LIST
#define FF_ATC_PAGE_LIST 1024
#endif
constexpr int MAX_PAGE_LIST = FF_ATC_PAGE_LIST;
static_assert(MAX_PAGE_LIST >= 16 && MAX_PAGE_LIST % 16 == 0, "two halves of whole tiles (up to 8 pages each)");
constexpr float LOG2E = 1.4426950408889634f;
constexpr unsigned long long WAIT_LIMIT_CYCLES = 2000000000ull;

constexpr int Q_BYTES = BM * D * 2;
constexpr int KV_TILE_BYTES = BN * D * 2;            // one K or V tile
// tensor memory: S in two buffers of BN columns (P, as bfloat16 pairs, takes the first BN/2
// columns of the S it was computed from), then O
constexpr int TMEM_COLS = (2 * BN + D) <= 256 ? 256 : 512;
constexpr size_t ATC_SMEM = 1024 + Q_BYTES + KV_STAGES * 2 * KV_TILE_BYTES + 128 + MAX_PAGE_LIST * 4;
// barriers
enum { B_K_FULL = 0, B_V_FULL = 2, B_K_EMPTY = 4, B_V_EMPTY = 6, B_S_FULL = 8, B_P_FULL = 10, B_PV_DONE = 12,
       B_Q_READY = 13, B_PAGES_READY = 14, B_COUNT = 15 };
// S and P have a barrier per buffer: a softmax warp may be a whole tile ahead of another, and its
// arrival for the next tile must not count for this one

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
        __nanosleep(32);                     // leave the issue slots to the warps that have work
        if (((++spins) & 1023u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - start > WAIT_LIMIT_CYCLES) {
                atomicExch(status, 107);
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
__device__ __forceinline__ void tc_commit_to(bool issue, uint32_t bar) {
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
                 "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
                 ::"r"(bar), "r"((uint32_t)issue) : "memory");
}
// The MMA warp runs its loop with all lanes (so that descriptors and addresses are warp-uniform values);
// `issue` is true in the one lane that really issues the instruction.
__device__ __forceinline__ void tc_mma(bool issue, uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                 "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(acc), "r"((uint32_t)issue) : "memory");
}
// the same with the A operand (128 x 16 bfloat16, two to a 32-bit cell, 8 columns) in tensor memory
__device__ __forceinline__ void tc_mma_a_tmem(bool issue, uint32_t d_tmem, uint32_t a_tmem, uint64_t db, uint32_t idesc,
                                              uint32_t acc) {
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                 "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(db), "r"(idesc), "r"(acc), "r"((uint32_t)issue) : "memory");
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
// 32 consecutive accumulator columns of this warp's 32 lanes (no wait: call tm_ld_wait() before use)
__device__ __forceinline__ void tm_ld32_nowait(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void tm_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float fast_exp2(float x) {   // 2^x; -inf -> 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 2^x for two values, each exponential in 32-bit and only the result rounded to bfloat16 (the form
// P is stored in).  The argument must not be rounded to bfloat16 first: the reference max trails the
// true max by up to 8, so the heaviest keys have arguments in [4, 8), where bfloat16 is 2^-5 apart,
// about 1 % in the weight; that is several times the rounding of P itself.
__device__ __forceinline__ uint32_t exp2_bf16x2(float x0, float x1) {
    uint32_t y;
    const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(y) : "f"(p1), "f"(p0));        // low half = p0
    return y;
}
__device__ __forceinline__ void tm_st16(uint32_t taddr, const float (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
                   "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
                   "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])),
                   "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
                   "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
                   "r"(__float_as_uint(v[15])) : "memory");
}

__device__ __forceinline__ void tm_st16u(uint32_t taddr, const uint32_t* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
                   "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}

// Operand descriptors.  Tiles are made of 64-column panels whose 128-byte rows are swizzled in
// groups of eight (the layout TMA writes with the 128-byte swizzle).
// K-major (the reduction dimension runs along the 128-byte row): groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// N-major (the rows of the tile are the reduction dimension, the 128-byte row runs along N):
// groups of 8 reduction rows 1024 bytes apart (stride offset), 64-column panels `panel_bytes`
// apart (leading offset).
__device__ __forceinline__ uint64_t desc_n_major(uint32_t addr, uint32_t panel_bytes) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)((panel_bytes >> 4) & 0x3FFF) << 16) |
           ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// bfloat16 x bfloat16 -> float32, M = 128, N = n; b_n_major: the B operand is N-major
__device__ __forceinline__ uint32_t idesc_bf16(int n, bool b_n_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_n_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(BM >> 4) << 24);
}

struct alignas(64) TensorMapArg { unsigned char bytes[128]; };   // a CUtensorMap, opaque to device code

__global__ void __launch_bounds__(ATC_THREADS)
attn_tc_kernel(const __grid_constant__ TensorMapArg kv_map, const bf16* __restrict__ q, int q_stride,
               const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_q,
               const int* __restrict__ ctx_lens, int n_seqs, bf16* __restrict__ out, int out_stride, int nq,
               int nkv, int block_size, int num_blocks, float scale_log2, int window, int* __restrict__ status,
               int num_splits, float* __restrict__ part_o, float* __restrict__ part_ml) {
    // num_splits > 1: the grid holds every (row tile, kv head) num_splits times; each copy walks its share
    // of the tile's keys and leaves an unnormalised result with its (reference max, sum) for the join
    // kernel.  For prompts so short that their row tiles would leave most SMs idle while each block
    // walks a long chain of key tiles alone.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* Qs = base;                                        // [PANELS][128][128 B]
    unsigned char* Ks = Qs + Q_BYTES;                                // [stage][PANELS][64][128 B]
    unsigned char* Vs = Ks + KV_STAGES * KV_TILE_BYTES;              // [stage][PANELS][64][128 B]
    uint64_t* bars = reinterpret_cast<uint64_t*>(Vs + KV_STAGES * KV_TILE_BYTES);
    int* s_pages = reinterpret_cast<int*>(bars + 16);
    __shared__ int s_seq, s_tile, s_abort, s_tok0, s_qlen, s_ctx;
    __shared__ uint32_t s_tmem;
    const int G = nq / nkv;
    const unsigned units = gridDim.x / (unsigned)num_splits;          // (row tile, kv head) pairs
    const unsigned unit = blockIdx.x % units;
    const int split = (int)(blockIdx.x / units);
    const int kh = (int)(unit % (unsigned)nkv);
    // the warp index through a shuffle, so that the compiler knows it to be the same in the whole warp and
    // keeps the address arithmetic of the single-thread roles in uniform registers
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    volatile int* abort_flag = &s_abort;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int i = 0; i < B_COUNT; ++i) mb_init(sa(&bars[i]), (i == B_P_FULL || i == B_P_FULL + 1 || i >= B_Q_READY) ? 4 : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(sa(&s_tmem)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // Row tiles are handed out last first, for all kv heads before the next tile: in a prompt the
    // late tiles see the most keys, and the long blocks should not be the ones that start last.
    const int vtile = (int)(units / (unsigned)nkv) - 1 - (int)(unit / (unsigned)nkv);
    if (warp == 0) {   // which sequence owns row tile vtile
        int cum = 0, found_seq = -1, found_tile = 0;
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
            const unsigned hit = __ballot_sync(0xffffffffu, cum + incl > vtile);
            if (hit) {
                const int l0 = __ffs(hit) - 1;
                found_seq = s0 + l0;
                found_tile = vtile - (cum + __shfl_sync(0xffffffffu, incl, l0) - __shfl_sync(0xffffffffu, cnt, l0));
            }
            cum += total;
        }
        if (lane == 0) {
            s_seq = found_seq; s_tile = found_tile;
            if (found_seq >= 0) {
                const int a = cu_q[found_seq];
                s_tok0 = a; s_qlen = cu_q[found_seq + 1] - a; s_ctx = ctx_lens[found_seq];
            }
        }
    }
    tc_before();
    __syncthreads();
    tc_after();
    const uint32_t tmem = s_tmem;
    const uint32_t tm_S = tmem;                  // two buffers: columns [0, 64) and [64, 128)
    const uint32_t tm_O = tmem + 2 * BN;         // columns [128, 128 + D)
    const int seq = s_seq, tile = s_tile;

    int n_tiles = 0, t_begin = 0, tok0 = 0, q_len = 0, ctx = 0, rows = 0, row0 = 0, kv_lo = 0, kv_hi = 0;
    if (seq >= 0) {
        tok0 = s_tok0; q_len = s_qlen; ctx = s_ctx;
        rows = q_len * G; row0 = tile * BM;
        const int first_tok = row0 / G, last_tok = min(q_len - 1, (row0 + BM - 1) / G);
        kv_hi = ctx + last_tok + 1;
        kv_lo = window > 0 ? max(0, ctx + first_tok - window + 1) : 0;
        t_begin = kv_lo / BN;
        n_tiles = (kv_hi + BN - 1) / BN - t_begin;
        if (num_splits > 1) {                    // this copy's share of the key tiles (it may be empty)
            const int per = (n_tiles + num_splits - 1) / num_splits;
            const int mine = min(per, max(0, n_tiles - split * per));
            t_begin += split * per;
            n_tiles = mine;
        }
    }
    const int pages_per_tile = BN / block_size;
    const int tiles_per_half = (MAX_PAGE_LIST / 2) / pages_per_tile;      // tiles whose page ids one half of the ring holds
    if (seq < 0) n_tiles = 0;
    // Page ids of tiles [first, first + count) of this block into their places of the ring, by the
    // threads `who` of `nthreads`.  A page that should be there and is not raises status 4.
    const int* bt = block_table + (size_t)max(seq, 0) * max_blocks;
    const int last_page = (kv_hi - 1) / block_size, first_page = kv_lo / block_size;
    auto fill_pages = [&](int first, int count, int who, int nthreads) {
        for (int i = who; i < count * pages_per_tile; i += nthreads) {
            const int tile = first + i / pages_per_tile;
            const int pi = (t_begin + tile) * pages_per_tile + i % pages_per_tile;
            const bool wanted = pi >= first_page && pi <= last_page;
            int page = (wanted && pi < max_blocks) ? bt[pi] : -1;
            if (page >= num_blocks) page = -1;
            if (wanted && page < 0) atomicExch(status, 4);      // a key's page is missing: the bookkeeping is at fault
            s_pages[(tile % (2 * tiles_per_half)) * pages_per_tile + i % pages_per_tile] = page;
        }
    };

    if (warp < 4) {
        // ------------------------------------------------ set-up by the softmax warps --
        const int r = threadIdx.x;                            // this thread's row of the tile
        const int rg = row0 + r;
        const bool valid = rg < rows;
        const int rgc = min(rg, max(rows - 1, 0));
        const int token = rgc / G, head = kh * G + rgc % G;
        // this row of q into registers first: its latency passes under the work on the page list
        uint4 qv[D / 8];
        if (n_tiles > 0) {
            const uint4* src = reinterpret_cast<const uint4*>(q + (size_t)(tok0 + token) * q_stride + (size_t)head * D);
#pragma unroll
            for (int ch = 0; ch < D / 8; ++ch) qv[ch] = valid ? __ldg(src + ch) : make_uint4(0u, 0u, 0u, 0u);
        }
        // page ids of the first tiles (both halves of the ring)
        fill_pages(0, min(n_tiles, 2 * tiles_per_half), threadIdx.x, 128);
        // zero the K/V stages once: parts no page is loaded into must hold finite numbers
        for (int i = threadIdx.x; i < KV_STAGES * 2 * KV_TILE_BYTES / 16; i += 128)
            reinterpret_cast<uint4*>(Ks)[i] = make_uint4(0u, 0u, 0u, 0u);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mb_arrive(sa(&bars[B_PAGES_READY]));               // the loads may start
        // the row of q -> the swizzled Q tile
        if (n_tiles > 0) {
#pragma unroll
            for (int ch = 0; ch < D / 8; ++ch)
                *reinterpret_cast<uint4*>(Qs + (ch >> 3) * (BM * 128) + r * 128 + (((ch & 7) ^ (r & 7)) << 4)) = qv[ch];
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mb_arrive(sa(&bars[B_Q_READY]));

        // ------------------------------------------------ softmax, one thread per row --
        const int pos = ctx + token;
        const int hi = pos + 1;
        const int lo = window > 0 ? max(0, pos - window + 1) : 0;
        const int first_pos = ctx + row0 / G;                        // the tile's smallest position
        const int last_pos = ctx + min(q_len - 1, (row0 + BM - 1) / G);
        const int full_lo = window > 0 ? max(0, last_pos - window + 1) : 0;
        const uint32_t lane_base = (uint32_t)((warp * 32) << 16);
        float m = -CUDART_INF_F, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            ok = mb_wait(sa(&bars[B_S_FULL + (j & 1)]), (j >> 1) & 1, status, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_after();
            const uint32_t tm_Sj = tm_S + (uint32_t)((j & 1) * BN) + lane_base;
            const int key0 = (t_begin + j) * BN;
            const bool need_mask = key0 + BN > first_pos + 1 || key0 < full_lo;
            float s[BN];
            tm_ld32_nowait(tm_Sj, s);
            tm_ld32_nowait(tm_Sj + 32, s + 32);
            tm_ld_wait();
            // mask (only tiles that touch the diagonal or a window's edge), then the row max of the raw
            // scores with four independent chains; the scale (> 0) is applied later
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < BN; ++i) {
                    const int key = key0 + i;
                    if (key < lo || key >= hi) s[i] = -CUDART_INF_F;
                }
            }
            float mx4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
            for (int i = 4; i < BN; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], s[i]);
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
            // The reference max `m` follows the true row max lazily: it moves (and O is rescaled) only
            // when the true max has grown by more than 2^8 since, which keeps p <= 256 and makes the
            // rescale rare after the first tiles.
            float corr = 1.0f;
            if (mx > m + 8.0f || m == -CUDART_INF_F) {
                const float m_new = fmaxf(m, mx);
                const float msafe_new = m_new == -CUDART_INF_F ? 0.f : m_new;
                corr = fast_exp2(m - msafe_new);               // m = -inf: 0
                m = m_new;
            }
            const float neg_m = m == -CUDART_INF_F ? 0.f : -m;
            // p = 2^(s*scale - m) in 32-bit, rounded to bfloat16 in pairs; the row sum adds the rounded
            // values, the same numbers the P V product sees
            uint32_t w[BN / 2];
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int e = 0; e < BN / 2; ++e) {
                w[e] = exp2_bf16x2(fmaf(s[2 * e], scale_log2, neg_m), fmaf(s[2 * e + 1], scale_log2, neg_m));
                sum4[e & 3] += __uint_as_float(w[e] << 16) + __uint_as_float(w[e] & 0xffff0000u);
            }
            // Tensor memory is written only between products: the last P V must be complete before P
            // of this tile is stored (stores issued while it was still running gave wrong sums, although
            // they go to other columns), and before O is rescaled.  It was issued a whole tile ago.
            if (j > 0) {
                ok = mb_wait(sa(&bars[B_PV_DONE]), (j - 1) & 1, status, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_after();
                if (!__all_sync(0xffffffffu, corr == 1.0f)) {          // some row's reference max moved: rescale O
#pragma unroll 1
                    for (int c = 0; c < D / 32; ++c) {
                        float v[32];
                        tm_ld32_nowait(tm_O + lane_base + c * 32, v);
                        tm_ld_wait();
                        float lo16[16], hi16[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) { lo16[i] = v[i] * corr; hi16[i] = v[16 + i] * corr; }
                        tm_st16(tm_O + lane_base + c * 32, lo16);
                        tm_st16(tm_O + lane_base + c * 32 + 16, hi16);
                    }
                }
            }
            // P over the first half of this S buffer (the row's scores are in registers by now)
            tm_st16u(tm_Sj, w);
            tm_st16u(tm_Sj + 16, w + 16);
            l = l * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_before();
            __syncwarp();
            if (lane == 0) mb_arrive(sa(&bars[B_P_FULL + (j & 1)]));
        }
        // ------------------------------------------------ epilogue ------------
        if (n_tiles > 0 && ok) {
            ok = mb_wait(sa(&bars[B_PV_DONE]), (n_tiles - 1) & 1, status, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (num_splits > 1) {
            // the partial result of this share of the keys: O unnormalised in 32-bit, its reference max
            // (in powers of two) and sum; a share without keys says so with max = -inf
            if (n_tiles > 0 && ok) tc_after();
            const size_t p = ((size_t)(tok0 + token) * nq + head) * num_splits + split;
            const bool any = n_tiles > 0 && ok && l > 0.f;
            if (valid && seq >= 0) {
                part_ml[p * 2] = any ? m : -CUDART_INF_F;
                part_ml[p * 2 + 1] = any ? l : 0.f;
            }
            if (n_tiles > 0 && ok) {
#pragma unroll 1
                for (int c = 0; c < D / 16; ++c) {
                    float v[16];
                    tm_ld16(tm_O + lane_base + c * 16, v);
                    if (valid) {
                        float4* dst4 = reinterpret_cast<float4*>(part_o + p * D + c * 16);
#pragma unroll
                        for (int i = 0; i < 4; ++i) dst4[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                    }
                }
            }
        } else if (n_tiles > 0 && ok) {
            tc_after();
            const float inv = 1.0f / l;
            bf16* dst = out + (size_t)(tok0 + token) * out_stride + (size_t)head * D;
#pragma unroll 1
            for (int c = 0; c < D / 16; ++c) {
                float v[16];
                tm_ld16(tm_O + lane_base + c * 16, v);
                if (valid) {
                    uint32_t w[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        __nv_bfloat162 pp = __floats2bfloat162_rn(v[2 * i] * inv, v[2 * i + 1] * inv);
                        w[i] = *reinterpret_cast<uint32_t*>(&pp);
                    }
                    *reinterpret_cast<uint4*>(dst + c * 16) = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(dst + c * 16 + 8) = make_uint4(w[4], w[5], w[6], w[7]);
                }
            }
        }
    } else if (warp == 4) {
        // ------------------------------------------------ loads: K and V tiles by TMA --
        // The whole warp: a tile is pages_per_tile x PANELS boxes (at most 32), one per lane, since a
        // single thread needs well over a hundred cycles for each copy it starts.
        // The softmax warps write the page list and zero the stages first.
        // Order K0, K1, V0, K2, V1, ...: the order in which the MMAs need them and free their stages.
        bool ok = n_tiles == 0 || mb_wait(sa(&bars[B_PAGES_READY]), 0, status, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        const int p = lane / PANELS, h = lane % PANELS;                  // this lane's page and panel of a tile
        auto load_tile = [&](int j, int kv) -> bool {
            const int s = j % KV_STAGES;
            if (kv == 0 && j >= 2 * tiles_per_half && j % tiles_per_half == 0) {
                // the K loads run ahead of the V loads by one tile and have reached a half of the ring whose
                // tiles are all behind both: refill it with the next tiles' page ids
                fill_pages(j, min(tiles_per_half, n_tiles - j), lane, 32);
                __syncwarp();
            }
            bool fine = mb_wait(sa(&bars[(kv ? B_V_EMPTY : B_K_EMPTY) + s]), ((j / KV_STAGES) & 1) ^ 1, status, abort_flag);
            if (!__all_sync(0xffffffffu, fine)) return false;
            const int page = p < pages_per_tile ? s_pages[(j % (2 * tiles_per_half)) * pages_per_tile + p] : -1;
            const unsigned boxes = __ballot_sync(0xffffffffu, page >= 0);
            const uint32_t bar = sa(&bars[(kv ? B_V_FULL : B_K_FULL) + s]);
            if (lane == 0) mb_expect_tx(bar, (uint32_t)(__popc(boxes) * block_size * 128));
            __syncwarp();
            if (page >= 0) {
                unsigned char* st = (kv ? Vs : Ks) + (size_t)s * KV_TILE_BYTES;
                const int y = ((page * 2 + kv) * nkv + kh) * block_size;
                tma_2d(sa(st + h * (BN * 128) + p * block_size * 128), &kv_map, h * 64, y, bar);
            }
            return true;
        };
        if (ok && n_tiles > 0) ok = load_tile(0, 0);
        for (int j = 0; j < n_tiles && ok; ++j) {
            if (j + 1 < n_tiles) ok = load_tile(j + 1, 0);
            if (ok) ok = load_tile(j, 1);
        }
    } else if (warp == 5) {
        // ------------------------------------------------ MMAs -----------------
        const uint32_t idesc_qk = idesc_bf16(BN, false);
        const uint32_t idesc_pv = idesc_bf16(D, true);
        const bool issue = lane == 0;                               // always the same lane: commits follow its MMAs
        bool ok = n_tiles == 0 || mb_wait(sa(&bars[B_Q_READY]), 0, status, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        tc_after();
        // S(j) = Q K(j)^T over D in steps of 16, into S buffer j & 1
        auto issue_qk = [&](int j) -> bool {
            const int s = j % KV_STAGES;
            if (!__all_sync(0xffffffffu, mb_wait(sa(&bars[B_K_FULL + s]), (j / KV_STAGES) & 1, status, abort_flag))) return false;
            tc_after();
            const uint32_t ks = sa(Ks + (size_t)s * KV_TILE_BYTES);
#pragma unroll
            for (int k = 0; k < D / 16; ++k) {
                const uint64_t da = desc_k_major(sa(Qs) + (k >> 2) * (BM * 128) + (k & 3) * 32);
                const uint64_t db = desc_k_major(ks + (k >> 2) * (BN * 128) + (k & 3) * 32);
                tc_mma(issue, tm_S + (uint32_t)((j & 1) * BN), da, db, idesc_qk, k > 0 ? 1u : 0u);
            }
            tc_commit_to(issue, sa(&bars[B_S_FULL + (j & 1)]));
            tc_commit_to(issue, sa(&bars[B_K_EMPTY + s]));
            __syncwarp();
            return true;
        };
        if (ok && n_tiles > 0) ok = issue_qk(0);
        for (int j = 0; j < n_tiles && ok; ++j) {
            // the next tile's scores first: they are computed while the softmax warps work on this tile
            if (j + 1 < n_tiles) {
                ok = issue_qk(j + 1);
                if (!ok) break;
            }
            const int s = j % KV_STAGES;
            // O += P V over the 64 keys in steps of 16, once the softmax warps have written P
            ok = __all_sync(0xffffffffu, mb_wait(sa(&bars[B_P_FULL + (j & 1)]), (j >> 1) & 1, status, abort_flag));
            if (!ok) break;
            ok = __all_sync(0xffffffffu, mb_wait(sa(&bars[B_V_FULL + s]), (j / KV_STAGES) & 1, status, abort_flag));
            if (!ok) break;
            tc_after();
            const uint32_t vs = sa(Vs + (size_t)s * KV_TILE_BYTES);
#pragma unroll
            for (int k = 0; k < BN / 16; ++k) {
                const uint64_t db = desc_n_major(vs + k * 16 * 128, BN * 128);
                tc_mma_a_tmem(issue, tm_O, tm_S + (uint32_t)((j & 1) * BN + k * 8), db, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
            }
            tc_commit_to(issue, sa(&bars[B_PV_DONE]));
            tc_commit_to(issue, sa(&bars[B_V_EMPTY + s]));
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

// Join of the shares: out[token, head, :] = sum_s w_s O_s / sum_s w_s l_s, w_s = 2^(m_s - max m), in
// the order of the shares.  D / 4 threads own one (token, head) and four columns each (16-byte loads,
// all shares' loads in flight together); a block of JOIN_THREADS takes as many pairs as fit it.
constexpr int JOIN_THREADS = 256;
constexpr int JOIN_MAX_SPLITS = 8;
__global__ void __launch_bounds__(JOIN_THREADS)
attn_tc_join_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                    bf16* __restrict__ out, int out_stride, int nq, int num_splits, int tok_base, int n_pairs) {
    asm volatile("griddepcontrol.launch_dependents;\n\tgriddepcontrol.wait;" ::: "memory");
    constexpr int TPP = D / 4;                                  // threads per (token, head)
    const int pair = blockIdx.x * (JOIN_THREADS / TPP) + threadIdx.x / TPP;
    if (pair >= n_pairs) return;
    const int col = (threadIdx.x % TPP) * 4;
    const int tok = tok_base + pair / nq, head = pair % nq;
    const size_t base = ((size_t)tok * nq + head) * num_splits;
    float ms[JOIN_MAX_SPLITS], ls[JOIN_MAX_SPLITS];
    float4 o[JOIN_MAX_SPLITS];
    float M = -CUDART_INF_F;
#pragma unroll
    for (int s = 0; s < JOIN_MAX_SPLITS; ++s) {
        if (s < num_splits) {
            const float2 ml = *reinterpret_cast<const float2*>(part_ml + (base + s) * 2);
            ms[s] = ml.x;
            ls[s] = ml.y;
            o[s] = *reinterpret_cast<const float4*>(part_o + (base + s) * D + col);
            M = fmaxf(M, ml.x);
        }
    }
    float L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < JOIN_MAX_SPLITS; ++s) {
        if (s < num_splits && ms[s] != -CUDART_INF_F) {
            const float w = exp2f(ms[s] - M);
            L += w * ls[s];
            acc.x += w * o[s].x; acc.y += w * o[s].y; acc.z += w * o[s].z; acc.w += w * o[s].w;
        }
    }
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    __align__(8) bf16 r[4] = {__float2bfloat16_rn(acc.x * inv), __float2bfloat16_rn(acc.y * inv),
                              __float2bfloat16_rn(acc.z * inv), __float2bfloat16_rn(acc.w * inv)};
    *reinterpret_cast<uint2*>(out + (size_t)tok * out_stride + (size_t)head * D + col) = *reinterpret_cast<const uint2*>(r);
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

// Tensor map of a cache slot seen as [rows, D] bfloat16: boxes of block_size rows x 64 columns, 128-byte swizzle.
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

FF_EXPORT int ff_attn_tc_block_m() { return BM; }

// total_tiles = sum over sequences of ceil(q_len * G / 128).  Needs a block size that divides 64
// (8, 16, 32 or 64), a 128-byte aligned cache and q rows aligned to 16 bytes.
// num_splits > 1: every row tile's keys are shared out over that many blocks, which leave partial
// results in part_o (float [tokens * nq * num_splits * D]) and part_ml (float [tokens * nq * num_splits * 2]),
// indexed by the token's row in q/out; a second kernel joins them for the n_tokens rows from tok_base on
// (the rows of the sequences given here).
FF_EXPORT int ff_attn_tc(const void* q, int q_stride, const void* cache, const int* block_table, int max_blocks,
                         const int* cu_q, const int* ctx_lens, int n_seqs, int total_tiles, void* out,
                         int out_stride, int nq, int nkv, int block_size, int num_blocks, float scale, int window,
                         int* status, int num_splits, float* part_o, float* part_ml, int tok_base, int n_tokens,
                         cudaStream_t stream) {
    if (n_seqs <= 0 || total_tiles <= 0) return 0;
    if (nkv <= 0 || nq % nkv) return FF_ERR_BAD_ARG;
    if (num_splits < 1 || (num_splits > 1 && (!part_o || !part_ml || n_tokens <= 0 || tok_base < 0))) return FF_ERR_BAD_ARG;
    if (num_splits > JOIN_MAX_SPLITS) return FF_ERR_UNSUPPORTED;
    if (block_size < 8 || BN % block_size) return FF_ERR_UNSUPPORTED;
    if (((uintptr_t)cache & 127) || ((uintptr_t)q & 15) || (q_stride % 8) || ((uintptr_t)out & 15) || (out_stride % 8))
        return FF_ERR_UNSUPPORTED;
    const long long rows = (long long)num_blocks * 2 * nkv * block_size;
    if (rows >= (1ll << 31)) return FF_ERR_UNSUPPORTED;
    FF_SMEM_LIMIT(attn_tc_kernel, ATC_SMEM);
    CUtensorMap map;
    int rc = cache_map(cache, rows, block_size, &map);
    if (rc) return rc;
    TensorMapArg arg;
    std::memcpy(arg.bytes, &map, sizeof(map));
    if ((long long)total_tiles * nkv * num_splits >= (1ll << 31)) return FF_ERR_UNSUPPORTED;
    FF_LAUNCH((attn_tc_kernel), dim3((unsigned)(total_tiles * nkv * num_splits)), ATC_THREADS, ATC_SMEM, stream, arg,
              (const bf16*)q, q_stride, block_table, max_blocks, cu_q, ctx_lens, n_seqs, (bf16*)out, out_stride, nq, nkv,
              block_size, num_blocks, scale * LOG2E, window, status, num_splits, part_o, part_ml);
    if (num_splits > 1) {
        const int n_pairs = n_tokens * nq, per_block = JOIN_THREADS / (D / 4);
        FF_LAUNCH((attn_tc_join_kernel), dim3((unsigned)((n_pairs + per_block - 1) / per_block)), JOIN_THREADS, 0, stream,
                  (const float*)part_o, (const float*)part_ml, (bf16*)out, out_stride, nq, num_splits, tok_base, n_pairs);
        FF_LAUNCH_CHECK();
    }
    return 0;
}
