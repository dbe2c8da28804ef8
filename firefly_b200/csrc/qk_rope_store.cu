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

// The same for long portions of prompts, where the kernel is a stream over the projection's output:
// a lane owns eight consecutive elements of a head's lower half and the eight that rotate with them in
// the upper half (16-byte loads and stores), LPH = head size / 16 lanes make up a head, a warp takes
// HPW consecutive heads of one token in passes of 32 / LPH heads, with all its loads in flight
// together.  The token's position, page, cosines and sines are fetched once for all of them.
template <int LPH, int HPW>
__global__ void qk_norm_rope_store_rows_kernel(
    bf16* __restrict__ qkv, int row_width, int T_tokens, int nq, int nkv,
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
    const float* __restrict__ cos_sin, int max_positions,
    const int* __restrict__ positions, const int* __restrict__ token_seq,
    const int* __restrict__ block_table, int max_blocks, int block_size, int num_blocks,
    bf16* __restrict__ cache, int* __restrict__ status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int d = LPH * 16, HALF = d / 2, HPP = 32 / LPH, PASSES = HPW / HPP;
    static_assert(HPW % HPP == 0, "a warp's heads come in whole passes");
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane % LPH, hsel = lane / LPH;
    const int heads = nq + 2 * nkv;
    const int chunks = (heads + HPW - 1) / HPW;
    const long long item = (long long)blockIdx.x * QKR_WARPS + warp;
    const bool active = item < (long long)T_tokens * chunks;
    const int t = active ? (int)(item / chunks) : 0, h0 = active ? (int)(item % chunks) * HPW : 0;
    const int pos = positions[t];
    const int e0 = sub * 8;
    const bool pos_ok = pos >= 0 && pos < max_positions;
    float cs_c[8], cs_s[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { cs_c[j] = 1.f; cs_s[j] = 0.f; }
    if (cos_sin && pos_ok) {
        const float4* cs = reinterpret_cast<const float4*>(cos_sin + (size_t)pos * d + 2 * e0);   // [half][2]
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float4 v = __ldg(cs + j);
            cs_c[2 * j] = v.x; cs_s[2 * j] = v.y; cs_c[2 * j + 1] = v.z; cs_s[2 * j + 1] = v.w;
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
    uint4 a[PASSES], b[PASSES];
#pragma unroll
    for (int p = 0; p < PASSES; ++p) {
        const int hh = min(h0 + p * HPP + hsel, heads - 1);
        a[p] = *reinterpret_cast<const uint4*>(row + (size_t)hh * d + e0);
        b[p] = *reinterpret_cast<const uint4*>(row + (size_t)hh * d + HALF + e0);
    }
#pragma unroll
    for (int p = 0; p < PASSES; ++p) {
        const int hh = h0 + p * HPP + hsel;
        const bool valid = hh < heads;
        const int kind = hh < nq ? 0 : (hh < nq + nkv ? 1 : 2);  // q, k, v
        float lo[8], hi[8];
        const bf16* pa = reinterpret_cast<const bf16*>(&a[p]);
        const bf16* pb = reinterpret_cast<const bf16*>(&b[p]);
#pragma unroll
        for (int j = 0; j < 8; ++j) { lo[j] = __bfloat162float(pa[j]); hi[j] = __bfloat162float(pb[j]); }
        const float* nw = kind == 0 ? q_norm_w : (kind == 1 ? k_norm_w : nullptr);
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += lo[j] * lo[j] + hi[j] * hi[j];
#pragma unroll
        for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // over the head's lanes
        if (nw) {
            const float inv = 1.0f / sqrtf(ss / (float)d + eps);
            const float4* wl = reinterpret_cast<const float4*>(nw + e0);
            const float4* wh = reinterpret_cast<const float4*>(nw + HALF + e0);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float4 l = __ldg(wl + j), h = __ldg(wh + j);
                lo[4 * j] *= inv * l.x; lo[4 * j + 1] *= inv * l.y; lo[4 * j + 2] *= inv * l.z; lo[4 * j + 3] *= inv * l.w;
                hi[4 * j] *= inv * h.x; hi[4 * j + 1] *= inv * h.y; hi[4 * j + 2] *= inv * h.z; hi[4 * j + 3] *= inv * h.w;
            }
        }
        if (kind != 2 && cos_sin) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float x = lo[j], y = hi[j];
                lo[j] = x * cs_c[j] - y * cs_s[j];
                hi[j] = y * cs_c[j] + x * cs_s[j];
            }
        }
        if (!valid) continue;
        bf16* dst = row + (size_t)hh * d;
        if (kind != 0) {
            const int kh = kind == 1 ? hh - nq : hh - nq - nkv;
            dst = cache + ((((size_t)page * 2 + (kind == 2)) * nkv + kh) * block_size + pos % block_size) * d;
        }
        uint4 oa, ob;
        bf16* qa = reinterpret_cast<bf16*>(&oa);
        bf16* qb = reinterpret_cast<bf16*>(&ob);
#pragma unroll
        for (int j = 0; j < 8; ++j) { qa[j] = __float2bfloat16_rn(lo[j]); qb[j] = __float2bfloat16_rn(hi[j]); }
        *reinterpret_cast<uint4*>(dst + e0) = oa;
        *reinterpret_cast<uint4*>(dst + HALF + e0) = ob;
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
        const bool wide_ok = row_width % 8 == 0 && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)cache & 15) == 0 &&
                             ((uintptr_t)cos_sin & 15) == 0 && ((uintptr_t)q_norm_w & 15) == 0 && ((uintptr_t)k_norm_w & 15) == 0;
        if (T >= 256 && wide_ok) {   // long portions: a warp per (token, 8 heads), 16 bytes a lane
            constexpr int HPW = 8;
            const long long ritems = (long long)T * ((nq + 2 * nkv + HPW - 1) / HPW);
            const unsigned rblocks = (unsigned)((ritems + QKR_WARPS - 1) / QKR_WARPS);
            if (d == 128)
                FF_LAUNCH((qk_norm_rope_store_rows_kernel<8, HPW>), rblocks, QKR_WARPS * 32, 0, stream, (bf16*)qkv,
                          row_width, T, nq, nkv, q_norm_w, k_norm_w, eps, cos_sin, max_positions, positions, token_seq,
                          block_table, max_blocks, block_size, num_blocks, (bf16*)cache, status);
            else
                FF_LAUNCH((qk_norm_rope_store_rows_kernel<16, HPW>), rblocks, QKR_WARPS * 32, 0, stream, (bf16*)qkv,
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
