// Per-head RMSNorm of q and k, rotary position encoding, and the write of k and v
// into the paged cache, in one pass over the projection's output.
//
// The reference does this in four launches: two rms_norm calls with a row = one
// head (src/model/qwen_model.cu:124-128), apply_rope (src/kernels/rope.cu:22-137)
// and append_kv_cache (src/model/qwen_model.cu:21-47).  Here one warp owns one
// (token, head): it normalises in 32-bit, rotates with cosines and sines taken from
// a table built on the host in double precision, and rounds once on the way out.
// q is rewritten in place; k (normalised, rotated) and v (raw) go to their page.
//
// Cache layout of one slot: [num_blocks][2 (k,v)][n_kv_heads][block_size][head_dim].
#include "common.cuh"

#include <type_traits>

namespace ff {

constexpr int QKR_WARPS = 4;
constexpr int QKR_MAX_D = 256;

template <typename T>
__global__ void qk_norm_rope_store_kernel(
    T* __restrict__ qkv, int row_width, int T_tokens, int nq, int nkv, int d,
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
    const float* __restrict__ cos_sin, int rotary_dim, int max_positions,
    const int* __restrict__ positions, const int* __restrict__ token_seq,
    const int* __restrict__ block_table, int max_blocks, int block_size, int num_blocks,
    T* __restrict__ cache, int* __restrict__ status) {
    pdl_prologue();
    __shared__ float bufs[QKR_WARPS][QKR_MAX_D];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int heads = nq + 2 * nkv;
    const long long item = (long long)blockIdx.x * QKR_WARPS + warp;
    if (item >= (long long)T_tokens * heads) return;
    const int t = (int)(item / heads), hh = (int)(item % heads);
    float* buf = bufs[warp];
    T* src = qkv + (size_t)t * row_width + (size_t)hh * d;
    const int kind = hh < nq ? 0 : (hh < nq + nkv ? 1 : 2);  // q, k, v
    const int pos = positions[t];

    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
        float v = to_float(src[i]);
        buf[i] = v;
        ss += v * v;
    }
    const float* nw = kind == 0 ? q_norm_w : (kind == 1 ? k_norm_w : nullptr);
    if (nw) {
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)d + eps);
        for (int i = lane; i < d; i += 32) buf[i] = buf[i] * inv * nw[i];
    }
    __syncwarp();

    T* dst = src;
    if (kind != 0) {
        const int seq = token_seq[t];
        const int page = (pos >= 0 && pos / block_size < max_blocks) ? block_table[(size_t)seq * max_blocks + pos / block_size] : -1;
        if (page < 0 || page >= num_blocks) {
            if (lane == 0) atomicExch(status, 2);
            return;
        }
        const int kh = kind == 1 ? hh - nq : hh - nq - nkv;
        dst = cache + ((((size_t)page * 2 + (kind == 2)) * nkv + kh) * block_size + pos % block_size) * d;
    }
    if (kind != 2 && cos_sin) {
        if (pos < 0 || pos >= max_positions) {
            if (lane == 0) atomicExch(status, 3);
            return;
        }
        const int half = rotary_dim / 2;
        const float* cs = cos_sin + (size_t)pos * rotary_dim;  // [half][2]
        for (int i = lane; i < half; i += 32) {
            const float c = cs[2 * i], s = cs[2 * i + 1];
            const float lo = buf[i], hi = buf[i + half];
            dst[i] = from_float<T>(lo * c - hi * s);
            dst[i + half] = from_float<T>(hi * c + lo * s);
        }
        for (int i = rotary_dim + lane; i < d; i += 32) dst[i] = from_float<T>(buf[i]);
    } else {
        for (int i = lane; i < d; i += 32) dst[i] = from_float<T>(buf[i]);
    }
}

// The same for bfloat16 with a head of 64*C elements that is rotated whole: a lane keeps C
// consecutive elements of the first half and the C they pair with in the second half in registers,
// so every access of the warp is one full line and nothing goes through shared memory.
template <int C>
__global__ void qk_norm_rope_store_vec_kernel(
    bf16* __restrict__ qkv, int row_width, int T_tokens, int nq, int nkv,
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
    const float* __restrict__ cos_sin, int max_positions,
    const int* __restrict__ positions, const int* __restrict__ token_seq,
    const int* __restrict__ block_table, int max_blocks, int block_size, int num_blocks,
    bf16* __restrict__ cache, int* __restrict__ status) {
    // Only the projection's output depends on the kernel in front: position, page, norm weights,
    // cosines and sines are fetched before the wait for it.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int HALF = 32 * C, d = 64 * C;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int heads = nq + 2 * nkv;
    const long long item = (long long)blockIdx.x * QKR_WARPS + warp;
    const bool active = item < (long long)T_tokens * heads;
    const int t = active ? (int)(item / heads) : 0, hh = active ? (int)(item % heads) : 0;
    bf16* src = qkv + (size_t)t * row_width + (size_t)hh * d;
    const int kind = hh < nq ? 0 : (hh < nq + nkv ? 1 : 2);  // q, k, v
    const int pos = positions[t];
    const int e0 = lane * C;                                  // this lane's first element of each half
    const float* nw = kind == 0 ? q_norm_w : (kind == 1 ? k_norm_w : nullptr);
    float wl[C], wh[C], cs_c[C], cs_s[C];
#pragma unroll
    for (int j = 0; j < C; ++j) {
        wl[j] = nw ? nw[e0 + j] : 1.f;
        wh[j] = nw ? nw[HALF + e0 + j] : 1.f;
    }
    int page = 0;
    if (kind != 0) page = (pos >= 0 && pos / block_size < max_blocks) ? block_table[(size_t)token_seq[t] * max_blocks + pos / block_size] : -1;
    const bool rotate = kind != 2 && cos_sin != nullptr;
    const bool pos_ok = pos >= 0 && pos < max_positions;
#pragma unroll
    for (int j = 0; j < C; ++j) {
        cs_c[j] = 1.f;
        cs_s[j] = 0.f;
        if (rotate && pos_ok) {
            const float* cs = cos_sin + (size_t)pos * d + 2 * (e0 + j);  // [half][2]
            cs_c[j] = cs[0];
            cs_s[j] = cs[1];
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (!active) return;

    float lo[C], hi[C];
    {
        __align__(8) bf16 a[C], b[C];
        if (C == 2) {
            *reinterpret_cast<uint32_t*>(a) = *reinterpret_cast<const uint32_t*>(src + e0);
            *reinterpret_cast<uint32_t*>(b) = *reinterpret_cast<const uint32_t*>(src + HALF + e0);
        } else {
            *reinterpret_cast<uint2*>(a) = *reinterpret_cast<const uint2*>(src + e0);
            *reinterpret_cast<uint2*>(b) = *reinterpret_cast<const uint2*>(src + HALF + e0);
        }
#pragma unroll
        for (int j = 0; j < C; ++j) { lo[j] = __bfloat162float(a[j]); hi[j] = __bfloat162float(b[j]); }
    }
    if (nw) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < C; ++j) ss += lo[j] * lo[j] + hi[j] * hi[j];
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
        for (int j = 0; j < C; ++j) {
            lo[j] = lo[j] * inv * wl[j];
            hi[j] = hi[j] * inv * wh[j];
        }
    }
    bf16* dst = src;
    if (kind != 0) {
        if (page < 0 || page >= num_blocks) {
            if (lane == 0) atomicExch(status, 2);
            return;
        }
        const int kh = kind == 1 ? hh - nq : hh - nq - nkv;
        dst = cache + ((((size_t)page * 2 + (kind == 2)) * nkv + kh) * block_size + pos % block_size) * d;
    }
    if (rotate) {
        if (!pos_ok) {
            if (lane == 0) atomicExch(status, 3);
            return;
        }
#pragma unroll
        for (int j = 0; j < C; ++j) {
            const float a = lo[j], b = hi[j];
            lo[j] = a * cs_c[j] - b * cs_s[j];
            hi[j] = b * cs_c[j] + a * cs_s[j];
        }
    }
    __align__(8) bf16 a[C], b[C];
#pragma unroll
    for (int j = 0; j < C; ++j) { a[j] = __float2bfloat16_rn(lo[j]); b[j] = __float2bfloat16_rn(hi[j]); }
    if (C == 2) {
        *reinterpret_cast<uint32_t*>(dst + e0) = *reinterpret_cast<const uint32_t*>(a);
        *reinterpret_cast<uint32_t*>(dst + HALF + e0) = *reinterpret_cast<const uint32_t*>(b);
    } else {
        *reinterpret_cast<uint2*>(dst + e0) = *reinterpret_cast<const uint2*>(a);
        *reinterpret_cast<uint2*>(dst + HALF + e0) = *reinterpret_cast<const uint2*>(b);
    }
}

// The same for long portions of prompts: a warp takes HPW consecutive heads of one token, so the
// token's position, page, cosines and sines are fetched once for all of them and the loads of the
// HPW heads are in flight together.
template <int C, int HPW>
__global__ void qk_norm_rope_store_rows_kernel(
    bf16* __restrict__ qkv, int row_width, int T_tokens, int nq, int nkv,
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
    const float* __restrict__ cos_sin, int max_positions,
    const int* __restrict__ positions, const int* __restrict__ token_seq,
    const int* __restrict__ block_table, int max_blocks, int block_size, int num_blocks,
    bf16* __restrict__ cache, int* __restrict__ status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int HALF = 32 * C, d = 64 * C;
    using Vec = typename std::conditional<C == 2, uint32_t, uint2>::type;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int heads = nq + 2 * nkv;
    const int chunks = (heads + HPW - 1) / HPW;
    const long long item = (long long)blockIdx.x * QKR_WARPS + warp;
    const bool active = item < (long long)T_tokens * chunks;
    const int t = active ? (int)(item / chunks) : 0, h0 = active ? (int)(item % chunks) * HPW : 0;
    const int pos = positions[t];
    const int e0 = lane * C;
    float wq_l[C], wq_h[C], wk_l[C], wk_h[C], cs_c[C], cs_s[C];
    const bool pos_ok = pos >= 0 && pos < max_positions;
#pragma unroll
    for (int j = 0; j < C; ++j) {
        wq_l[j] = q_norm_w ? q_norm_w[e0 + j] : 1.f;
        wq_h[j] = q_norm_w ? q_norm_w[HALF + e0 + j] : 1.f;
        wk_l[j] = k_norm_w ? k_norm_w[e0 + j] : 1.f;
        wk_h[j] = k_norm_w ? k_norm_w[HALF + e0 + j] : 1.f;
        cs_c[j] = 1.f;
        cs_s[j] = 0.f;
        if (cos_sin && pos_ok) {
            const float* cs = cos_sin + (size_t)pos * d + 2 * (e0 + j);  // [half][2]
            cs_c[j] = cs[0];
            cs_s[j] = cs[1];
        }
    }
    const bool has_kv = h0 + HPW > nq;
    int page = 0;
    if (has_kv) page = (pos >= 0 && pos / block_size < max_blocks) ? block_table[(size_t)token_seq[t] * max_blocks + pos / block_size] : -1;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (!active) return;
    if (has_kv && (page < 0 || page >= num_blocks)) {
        if (lane == 0) atomicExch(status, 2);
        return;
    }
    if (cos_sin && !pos_ok && h0 < nq + nkv) {
        if (lane == 0) atomicExch(status, 3);
        return;
    }
    bf16* row = qkv + (size_t)t * row_width;
    Vec a[HPW], b[HPW];
#pragma unroll
    for (int u = 0; u < HPW; ++u) {
        const int hh = min(h0 + u, heads - 1);
        a[u] = *reinterpret_cast<const Vec*>(row + (size_t)hh * d + e0);
        b[u] = *reinterpret_cast<const Vec*>(row + (size_t)hh * d + HALF + e0);
    }
#pragma unroll
    for (int u = 0; u < HPW; ++u) {
        const int hh = h0 + u;
        if (hh >= heads) break;
        const int kind = hh < nq ? 0 : (hh < nq + nkv ? 1 : 2);  // q, k, v
        float lo[C], hi[C];
        const bf16* pa = reinterpret_cast<const bf16*>(&a[u]);
        const bf16* pb = reinterpret_cast<const bf16*>(&b[u]);
#pragma unroll
        for (int j = 0; j < C; ++j) { lo[j] = __bfloat162float(pa[j]); hi[j] = __bfloat162float(pb[j]); }
        if ((kind == 0 && q_norm_w) || (kind == 1 && k_norm_w)) {
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < C; ++j) ss += lo[j] * lo[j] + hi[j] * hi[j];
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
            for (int j = 0; j < C; ++j) {
                lo[j] = lo[j] * inv * (kind == 0 ? wq_l[j] : wk_l[j]);
                hi[j] = hi[j] * inv * (kind == 0 ? wq_h[j] : wk_h[j]);
            }
        }
        if (kind != 2 && cos_sin) {
#pragma unroll
            for (int j = 0; j < C; ++j) {
                const float x = lo[j], y = hi[j];
                lo[j] = x * cs_c[j] - y * cs_s[j];
                hi[j] = y * cs_c[j] + x * cs_s[j];
            }
        }
        bf16* dst = row + (size_t)hh * d;
        if (kind != 0) {
            const int kh = kind == 1 ? hh - nq : hh - nq - nkv;
            dst = cache + ((((size_t)page * 2 + (kind == 2)) * nkv + kh) * block_size + pos % block_size) * d;
        }
        Vec oa, ob;
        bf16* qa = reinterpret_cast<bf16*>(&oa);
        bf16* qb = reinterpret_cast<bf16*>(&ob);
#pragma unroll
        for (int j = 0; j < C; ++j) { qa[j] = __float2bfloat16_rn(lo[j]); qb[j] = __float2bfloat16_rn(hi[j]); }
        *reinterpret_cast<Vec*>(dst + e0) = oa;
        *reinterpret_cast<Vec*>(dst + HALF + e0) = ob;
    }
}

}  // namespace ff

using namespace ff;

// nkv may be 0: a run that only reads another layer's cache has q heads alone.
FF_EXPORT int ff_qk_norm_rope_store(void* qkv, int dtype, int row_width, int T, int nq, int nkv, int d,
                                    const float* q_norm_w, const float* k_norm_w, float eps,
                                    const float* cos_sin, int rotary_dim, int max_positions,
                                    const int* positions, const int* token_seq, const int* block_table,
                                    int max_blocks, int block_size, int num_blocks, void* cache,
                                    int* status, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || d > QKR_MAX_D) return FF_ERR_UNSUPPORTED;
    if (cos_sin && (rotary_dim <= 0 || rotary_dim > d || (rotary_dim & 1))) return FF_ERR_BAD_ARG;
    if (row_width < (nq + 2 * nkv) * d) return FF_ERR_BAD_ARG;
    const long long items = (long long)T * (nq + 2 * nkv);
    const unsigned blocks = (unsigned)((items + QKR_WARPS - 1) / QKR_WARPS);
    // whole-head rotation of a 128- or 256-wide bfloat16 head with aligned rows: the register form
    if (dtype == 1 && (d == 128 || d == 256) && (!cos_sin || rotary_dim == d) && row_width % 4 == 0 &&
        ((uintptr_t)qkv & 7) == 0 && ((uintptr_t)cache & 7) == 0) {
        if (T >= 256) {   // long portions: a warp per (token, 8 heads)
            constexpr int HPW = 8;
            const long long ritems = (long long)T * ((nq + 2 * nkv + HPW - 1) / HPW);
            const unsigned rblocks = (unsigned)((ritems + QKR_WARPS - 1) / QKR_WARPS);
            if (d == 128)
                FF_LAUNCH((qk_norm_rope_store_rows_kernel<2, HPW>), rblocks, QKR_WARPS * 32, 0, stream, (bf16*)qkv,
                          row_width, T, nq, nkv, q_norm_w, k_norm_w, eps, cos_sin, max_positions, positions, token_seq,
                          block_table, max_blocks, block_size, num_blocks, (bf16*)cache, status);
            else
                FF_LAUNCH((qk_norm_rope_store_rows_kernel<4, HPW>), rblocks, QKR_WARPS * 32, 0, stream, (bf16*)qkv,
                          row_width, T, nq, nkv, q_norm_w, k_norm_w, eps, cos_sin, max_positions, positions, token_seq,
                          block_table, max_blocks, block_size, num_blocks, (bf16*)cache, status);
            FF_LAUNCH_CHECK();
            return 0;
        }
        if (d == 128)
            FF_LAUNCH((qk_norm_rope_store_vec_kernel<2>), blocks, QKR_WARPS * 32, 0, stream, (bf16*)qkv, row_width, T,
                      nq, nkv, q_norm_w, k_norm_w, eps, cos_sin, max_positions, positions, token_seq, block_table,
                      max_blocks, block_size, num_blocks, (bf16*)cache, status);
        else
            FF_LAUNCH((qk_norm_rope_store_vec_kernel<4>), blocks, QKR_WARPS * 32, 0, stream, (bf16*)qkv, row_width, T,
                      nq, nkv, q_norm_w, k_norm_w, eps, cos_sin, max_positions, positions, token_seq, block_table,
                      max_blocks, block_size, num_blocks, (bf16*)cache, status);
        FF_LAUNCH_CHECK();
        return 0;
    }
    if (dtype == 0)
        FF_LAUNCH((qk_norm_rope_store_kernel<float>), blocks, QKR_WARPS * 32, 0, stream, 
            (float*)qkv, row_width, T, nq, nkv, d, q_norm_w, k_norm_w, eps, cos_sin, rotary_dim,
            max_positions, positions, token_seq, block_table, max_blocks, block_size, num_blocks,
            (float*)cache, status);
    else if (dtype == 1)
        FF_LAUNCH((qk_norm_rope_store_kernel<bf16>), blocks, QKR_WARPS * 32, 0, stream, 
            (bf16*)qkv, row_width, T, nq, nkv, d, q_norm_w, k_norm_w, eps, cos_sin, rotary_dim,
            max_positions, positions, token_seq, block_table, max_blocks, block_size, num_blocks,
            (bf16*)cache, status);
    else
        return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}
