// Device helpers of the DFlash2 draft's row work, shared by draft.cu and by the GEMM finishes of segments.cuh that carry
// a row stage (conv after its projection, head norm + RoPE + K/V append after qkv).
#pragma once

#include "draft.h"

namespace mk {

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// Sums of squares to about 2^-45 without f64 arithmetic (scarce on this part): a square is split exactly into its rounded
// value and the rounding error (fma), the running sum keeps the exact error of every addition in a second word (two-sum).
struct F2 {
    float hi, lo;
};
__device__ __forceinline__ void f2_add(F2& s, float x) {
    const float t = __fadd_rn(s.hi, x), bb = __fsub_rn(t, s.hi);
    s.lo = __fadd_rn(s.lo, __fadd_rn(__fsub_rn(s.hi, __fsub_rn(t, bb)), __fsub_rn(x, bb)));
    s.hi = t;
}
__device__ __forceinline__ void f2_add_sq(F2& s, float x) {
    const float p = __fmul_rn(x, x);
    f2_add(s, p);
    s.lo = __fadd_rn(s.lo, __fmaf_rn(x, x, -p));
}
__device__ __forceinline__ void f2_merge(F2& s, const F2& o) {
    f2_add(s, o.hi);
    s.lo = __fadd_rn(s.lo, o.lo);
}
__device__ __forceinline__ F2 warp_sum_f2(F2 v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        F2 other;
        other.hi = __shfl_xor_sync(0xffffffffu, v.hi, o);
        other.lo = __shfl_xor_sync(0xffffffffu, v.lo, o);
        f2_merge(v, other);
    }
    return v;
}
__device__ __forceinline__ double f2_value(const F2& s) { return (double)s.hi + (double)s.lo; }

// 1 / sqrt(x) as two correctly rounded f32 operations
__device__ __forceinline__ float rsqrt_exact(float x) { return __fdiv_rn(1.0f, __fsqrt_rn(x)); }

__device__ __forceinline__ void record_clamp(int* status, int site, long long v) {
    if (status != nullptr && atomicCAS(status, 0, 4) == 0) {
        status[1] = site;
        status[2] = (int)blockIdx.x;
        status[3] = (int)v;
    }
}

__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
    const uint4 u = *(const uint4*)p;
    const __nv_bfloat162* h = (const __nv_bfloat162*)&u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __low2float(h[i]);
        v[2 * i + 1] = __high2float(h[i]);
    }
}
__device__ __forceinline__ void store8(bf16* p, const float (&v)[8]) {
    uint4 u;
    __nv_bfloat162* h = (__nv_bfloat162*)&u;
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *(uint4*)p = u;
}
// ---- head norm + neox RoPE -----------------------------------------------------------------------------------------------------
// One warp per 128-wide head: lane l holds elements 2l, 2l + 1 of the low half and of the high half. `round_normed`: the
// block's q / k round the normed head to bf16 before the rotation, the context K does not.
__device__ __forceinline__ void head_norm_rope_vals(float (&v)[4], const bf16* w, float eps, const float* cos_sin, bool round_normed,
                                                    bf16* out, int lane) {
    F2 sq = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 4; ++i) f2_add_sq(sq, v[i]);
    const float ms = (float)(f2_value(warp_sum_f2(sq)) / 128.0);
    const float r = rsqrt_exact(__fadd_rn(ms, eps));
    const __nv_bfloat162 wl = *(const __nv_bfloat162*)(w + 2 * lane), wh = *(const __nv_bfloat162*)(w + 64 + 2 * lane);
    const float wv[4] = {__low2float(wl), __high2float(wl), __low2float(wh), __high2float(wh)};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[i] = __fmul_rn(__fmul_rn(v[i], r), wv[i]);
        if (round_normed) v[i] = bf16_round(v[i]);
    }
    const float2 c = *(const float2*)(cos_sin + 2 * lane), s = *(const float2*)(cos_sin + 64 + 2 * lane);
    const float lo0 = __fsub_rn(__fmul_rn(v[0], c.x), __fmul_rn(v[2], s.x)), lo1 = __fsub_rn(__fmul_rn(v[1], c.y), __fmul_rn(v[3], s.y));
    const float hi0 = __fadd_rn(__fmul_rn(v[2], c.x), __fmul_rn(v[0], s.x)), hi1 = __fadd_rn(__fmul_rn(v[3], c.y), __fmul_rn(v[1], s.y));
    *(__nv_bfloat162*)(out + 2 * lane) = __floats2bfloat162_rn(lo0, lo1);
    *(__nv_bfloat162*)(out + 64 + 2 * lane) = __floats2bfloat162_rn(hi0, hi1);
}
__device__ __forceinline__ void head_norm_rope(const bf16* x, const bf16* w, float eps, const float* cos_sin, bool round_normed,
                                               bf16* out, int lane) {
    const __nv_bfloat162 xl = *(const __nv_bfloat162*)(x + 2 * lane), xh = *(const __nv_bfloat162*)(x + 64 + 2 * lane);
    float v[4] = {__low2float(xl), __high2float(xl), __low2float(xh), __high2float(xh)};
    head_norm_rope_vals(v, w, eps, cos_sin, round_normed, out, lane);
}

__device__ __forceinline__ long long clamp_pos(long long p, long long rows, int* status, int site) {
    if (p < 0 || p >= rows) {
        record_clamp(status, site, p);
        p = p < 0 ? 0 : rows - 1;
    }
    return p;
}


// One 128-wide head of a block row of the draft's qkv (lane l holds elements 2l, 2l + 1 of each half): q heads are normed,
// rounded, rotated and stored; k heads the same into the K pool at the row's ring slot; v heads are copied into the V pool.
__device__ __forceinline__ void dqkv_head(const DQkvRowsArgs& a, int m, int head, float (&v)[4], long long P, int lane) {
    const long long pos = clamp_pos(P + m, a.rope_rows, a.status, 410);
    const size_t slot = (size_t)((P + m) % a.pool_rows + a.pool_rows) % a.pool_rows;
    if (head < a.qh) {
        head_norm_rope_vals(v, a.q_norm, a.eps, a.rope + pos * kDraftHeadDim, true, a.q_out + ((size_t)m * a.qh + head) * kDraftHeadDim, lane);
    } else if (head < a.qh + a.kvh) {
        head_norm_rope_vals(v, a.k_norm, a.eps, a.rope + pos * kDraftHeadDim, true,
                            a.k_pool + (slot * a.kvh + (head - a.qh)) * kDraftHeadDim, lane);
    } else {
        bf16* dst = a.v_pool + (slot * a.kvh + (head - a.qh - a.kvh)) * kDraftHeadDim;
        *(__nv_bfloat162*)(dst + 2 * lane) = __floats2bfloat162_rn(v[0], v[1]);
        *(__nv_bfloat162*)(dst + 64 + 2 * lane) = __floats2bfloat162_rn(v[2], v[3]);
    }
}

}  // namespace mk
