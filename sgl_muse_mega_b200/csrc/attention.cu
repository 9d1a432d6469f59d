// Paged bf16 KV decode attention of the verify window (GQA, head_dim 64), split over the keys.
//
// One CTA per (kv head, key split). The window's M rows times the G query heads of a kv head form R = M G query rows;
// warp w owns rows 16w .. 16w+15 (row r = token r / G, head r % G). Keys are visited in blocks of 64: K and V rows are
// gathered through the position-ordered page table with 16-byte cp.async copies into XOR-swizzled shared tiles (two
// stages), QK^T and PV run on mma.sync m16n8k16 with P rounded to bf16 and the row sums kept in f32, the soft max runs
// in the exp2 domain (scores x 0.125 log2 e) and every split leaves an unnormalised (m, l, O) partial. A second kernel
// merges the splits in split order, normalises, applies the per-head weightless RMS norm and the sigmoid gate.
//
// Masks (row at position q, key at position p): p <= q, and on sliding-window layers q - p <= window.
// Reference: sm103/kernels/attention.cuh:1043-1481 (the arithmetic contract), test/reference/muse_spark.py:289-314.
#include "stages.h"

namespace mk {

constexpr int kKeyBlock = 64;
constexpr float kScaleLog2e = 0.125f * 1.4426950408889634f;


__device__ __forceinline__ uint32_t lds32(const unsigned char* p) { return *(const uint32_t*)p; }

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(a));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// The key blocks the window's rows see, and the splits that share them: a launch has `a.splits` CTAs per kv head (sized for
// the longest context), of which the first min(splits, blocks) take a contiguous share of the blocks each; the others
// leave at once and the merge does not read their partials. Both kernels derive the same numbers from kv_len.
struct AttnSpan {
    int lo, nblk, eff;
};
__device__ __forceinline__ AttnSpan attn_span(const AttnArgs& a, int kv_len) {
    AttnSpan sp;
    const int n_ctx = kv_len - a.M;
    sp.lo = a.window > 0 ? max(0, n_ctx - a.window) : 0;
    sp.nblk = (kv_len - sp.lo + kKeyBlock - 1) / kKeyBlock;
    // up to 40 blocks (a sliding window) one block a split; beyond, at least two blocks a split: the merge's cost grows with
    // the number of partials (measured at 8 K keys: 131 splits of one block 28 us, 72 of two 25 us)
    sp.eff = min(a.splits, max(sp.nblk <= 40 ? sp.nblk : (sp.nblk + 1) / 2, 1));
    return sp;
}

__global__ void __launch_bounds__(256, 2) attn_split_kernel(const AttnArgs a) {
    __shared__ __align__(128) unsigned char Ks[2][kKeyBlock * 128];
    __shared__ __align__(128) unsigned char Vs[2][kKeyBlock * 128];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, kvhead = blockIdx.y;
    RT(5, 0)
    // Everything up to the wait reads what earlier steps (or kernels two or more back) left: the window's length and page
    // table, and the context's K / V rows. The first key block's context rows are requested here, under the predecessor's
    // tail; only the window's own rows (appended by the predecessor) and the queries wait.
    const int kv_len = *a.kv_len;
    const int n_ctx = kv_len - a.M;
    const AttnSpan span = attn_span(a, kv_len);
    if (split >= span.eff) return;  // more splits than key blocks: the merge reads the first `eff` partials only
    const int lo = span.lo, nblk = span.nblk;
    const int b0 = (int)((long long)split * nblk / span.eff), b1 = (int)((long long)(split + 1) * nblk / span.eff);
    // part 0: the whole block; 1: its context keys (p < n_ctx); 2: the rest (window keys, zero fill past kv_len)
    auto load_block = [&](int b, int st, int part) {
        const int p0 = lo + b * kKeyBlock;
        for (int i = tid; i < kKeyBlock * 8; i += blockDim.x) {
            const int key = i >> 3, c = i & 7, p = p0 + key;
            if ((part == 1 && p >= n_ctx) || (part == 2 && p < n_ctx)) continue;
            const bool ok = p < kv_len;
            const long long off = ok ? a.page_table[p] + (long long)kvhead * 128 + c * 16 : 0;
            const int d = key * 128 + ((c ^ (key & 7)) << 4);
            cp_async16(&Ks[st][d], a.k_cache + off, ok);
            cp_async16(&Vs[st][d], a.v_cache + off, ok);
        }
        cp_async_commit();
    };
    if (b0 < b1) load_block(b0, 0, 1);
    griddep_wait();
    RT(5, 1)

    // Q fragments of this warp's 16 rows (rows >= R are zero)
    const int r0 = warp * 16 + g, r1 = r0 + 8;
    uint32_t qa[4][4];
    {
        const int tq0 = r0 / a.G, tq1 = r1 / a.G;
        const bf16* q0 = a.qkv + (size_t)tq0 * a.qkv_row + (kvhead * a.G + r0 % a.G) * kHeadDim;
        const bf16* q1 = a.qkv + (size_t)tq1 * a.qkv_row + (kvhead * a.G + r1 % a.G) * kHeadDim;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            qa[kk][0] = r0 < a.R ? *(const uint32_t*)(q0 + 16 * kk + 2 * t) : 0u;
            qa[kk][1] = r1 < a.R ? *(const uint32_t*)(q1 + 16 * kk + 2 * t) : 0u;
            qa[kk][2] = r0 < a.R ? *(const uint32_t*)(q0 + 16 * kk + 8 + 2 * t) : 0u;
            qa[kk][3] = r1 < a.R ? *(const uint32_t*)(q1 + 16 * kk + 8 + 2 * t) : 0u;
        }
    }
    // a row's position and, for a token-tree window (draft.h: the table's depth and ancestor-mask words), the window rows it
    // sees: a chain's row t sits at n_ctx + t and sees every earlier row; a tree's row sits at n_ctx + its depth and sees
    // its ancestors
    const int tq0 = min(r0 / a.G, a.M - 1), tq1 = min(r1 / a.G, a.M - 1);
    const int posq0 = n_ctx + (a.tree != nullptr ? a.tree[16 + tq0] : r0 / a.G), posq1 = n_ctx + (a.tree != nullptr ? a.tree[16 + tq1] : r1 / a.G);
    const unsigned tmask0 = a.tree != nullptr ? (unsigned)a.tree[32 + tq0] : 0u, tmask1 = a.tree != nullptr ? (unsigned)a.tree[32 + tq1] : 0u;

    float o[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m0 = -1e30f, m1 = -1e30f, l0 = 0.f, l1 = 0.f;

    if (b0 < b1) load_block(b0, 0, 2);
    for (int b = b0; b < b1; ++b) {
        const int st = (b - b0) & 1;
        if (b + 1 < b1) {
            load_block(b + 1, st ^ 1, 0);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const unsigned char* K = Ks[st];
        const unsigned char* V = Vs[st];
        // S = Q K^T : 8 key tiles of 8
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
            const int key = 8 * j + g;
            const unsigned char* row = K + key * 128 + 4 * t;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const uint32_t kb0 = lds32(row + (((2 * kk) ^ (key & 7)) << 4));
                const uint32_t kb1 = lds32(row + (((2 * kk + 1) ^ (key & 7)) << 4));
                mma_bf16_16816(s[j], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], kb0, kb1);
            }
        }
        // masks, running max
        const int pbase = lo + b * kKeyBlock;
        float mx0 = -1e30f, mx1 = -1e30f;
        // a block of context keys that every row of the window sees whole (all of a global layer's but the last, all of a
        // sliding window's but the first and the last) needs no per-element masks
        const bool whole = pbase + kKeyBlock <= n_ctx && (a.window <= 0 || pbase + a.window >= n_ctx + a.M - 1);
        unsigned vis = 0xFFFFFFFFu;  // bit 4 j + c
        if (whole) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
#pragma unroll
                for (int c = 0; c < 4; ++c) s[j][c] *= kScaleLog2e;
                mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
                mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
            }
        } else {
            vis = 0u;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int p = pbase + 8 * j + 2 * t + (c & 1);
                    const int pq = (c & 2) ? posq1 : posq0;
                    const bool own = a.tree == nullptr ? p <= pq : (p < n_ctx || ((((c & 2) ? tmask1 : tmask0) >> (p - n_ctx)) & 1u));
                    const bool v = own && p < kv_len && (a.window <= 0 || p + a.window >= pq);
                    vis |= (v ? 1u : 0u) << (4 * j + c);
                    s[j][c] *= kScaleLog2e;
                    if (v) {
                        if (c & 2) mx1 = fmaxf(mx1, s[j][c]);
                        else mx0 = fmaxf(mx0, s[j][c]);
                    }
                }
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float sc0 = exp2f(m0 - mn0), sc1 = exp2f(m1 - mn1);
        m0 = mn0;
        m1 = mn1;
        l0 *= sc0;
        l1 *= sc1;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            o[j][0] *= sc0;
            o[j][1] *= sc0;
            o[j][2] *= sc1;
            o[j][3] *= sc1;
        }
        uint32_t pa[4][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float p0 = (vis >> (4 * j)) & 1u ? exp2f(s[j][0] - m0) : 0.f;
            const float p1 = (vis >> (4 * j + 1)) & 1u ? exp2f(s[j][1] - m0) : 0.f;
            const float p2 = (vis >> (4 * j + 2)) & 1u ? exp2f(s[j][2] - m1) : 0.f;
            const float p3 = (vis >> (4 * j + 3)) & 1u ? exp2f(s[j][3] - m1) : 0.f;
            l0 += p0 + p1;
            l1 += p2 + p3;
            pa[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
            pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        // O += P V : ldmatrix.trans gives V^T fragments; matrices: (keys 0-7 | 8-15) x (dims 8jd | 8(jd+1))
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int jd = 0; jd < 8; jd += 2) {
                const int mi = lane >> 3, rr = lane & 7;
                const int key = 16 * kk + (mi & 1) * 8 + rr;
                const int dc = jd + (mi >> 1);
                uint32_t v0, v1, v2, v3;
                ldmatrix_x4_trans(v0, v1, v2, v3, V + key * 128 + ((dc ^ (key & 7)) << 4));
                mma_bf16_16816(o[jd], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], v0, v1);
                mma_bf16_16816(o[jd + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], v2, v3);
            }
        }
        __syncthreads();
    }
    // row sums across the quad
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    float* w0 = a.ws + ((size_t)(kvhead * a.splits + split) * a.R + r0) * 66;
    float* w1 = a.ws + ((size_t)(kvhead * a.splits + split) * a.R + r1) * 66;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        if (r0 < a.R) *(float2*)(w0 + 8 * j + 2 * t) = make_float2(o[j][0], o[j][1]);
        if (r1 < a.R) *(float2*)(w1 + 8 * j + 2 * t) = make_float2(o[j][2], o[j][3]);
    }
    if (t == 0) {
        if (r0 < a.R) { w0[64] = m0; w0[65] = l0; }
        if (r1 < a.R) { w1[64] = m1; w1[65] = l1; }
    }
    RT(5, 2)
}

// Four warps per (token, query head), two pairs per CTA: each warp merges a contiguous quarter of the splits in split
// order, the quarters meet in shared memory in order; then normalise, RMS norm, sigmoid gate. (One warp per pair walked
// up to 16 dependent batches of loads; the quarter walks at most 4.)
__global__ void __launch_bounds__(256) attn_combine_kernel(const AttnArgs a) {
    __shared__ float s_o[2][4][64];
    RT(6, 0)
    const int pc = threadIdx.x >> 7, wq = (threadIdx.x >> 5) & 3, lane = threadIdx.x & 31;
    const int w = blockIdx.x * 2 + pc;
    const bool valid = w < a.M * a.qh;
    const int tok = valid ? w / a.qh : 0, head = valid ? w % a.qh : 0;
    // the gate values sit in the qkv row the split kernel already waited for: requested before this kernel's own wait
    const bf16* og = a.qkv + (size_t)tok * a.qkv_row + (a.qh + 2 * a.kvh) * kHeadDim + head * kHeadDim + 2 * lane;
    const __nv_bfloat162 og2 = *(const __nv_bfloat162*)og;
    griddep_wait();
    griddep_launch();
    RT(6, 1)
    const int kvhead = head / a.G, r = tok * a.G + head % a.G;
    const float* base = a.ws + ((size_t)kvhead * a.splits * a.R + r) * 66;
    const size_t stride = (size_t)a.R * 66;
    // the (m, l) pairs of the splits live in the lanes (split s in lane s % 32, register s / 32): all loads independent
    constexpr int kPer = 8;  // splits <= 256
    const int n_splits = attn_span(a, *a.kv_len).eff;
    float ms_[kPer], ls_[kPer];
    float mx = -1e30f;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
        const int s = lane + 32 * i;
        ms_[i] = -1e30f;
        ls_[i] = 0.f;
        if (valid && s < n_splits) {
            const float2 ml = *(const float2*)(base + s * stride + 64);
            ms_[i] = ml.x;
            ls_[i] = ml.y;
        }
        mx = fmaxf(mx, ms_[i]);
    }
    mx = warp_max(mx);
    float L = 0.f;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
        ms_[i] = ls_[i] == 0.f ? 0.f : exp2f(ms_[i] - mx);  // now the split's scale (0 for an empty split)
        L += ls_[i] * ms_[i];
    }
    L = warp_sum(L);
    // this warp's quarter: O = sum over its splits, in split order, of O_s x scale_s: 8 independent loads per batch
    const int quarter = ((n_splits + 3) / 4 + 7) / 8 * 8, q0 = wq * quarter, q1 = min(q0 + quarter, n_splits);
    float o0 = 0.f, o1 = 0.f;
    for (int s0 = q0; s0 < q1; s0 += 8) {
        float2 v[8];
        float sc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int s = s0 + j;
            float scj = 0.f;
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                const float t = __shfl_sync(0xffffffffu, ms_[i], s & 31);
                if (i == (s >> 5)) scj = t;
            }
            sc[j] = s < q1 ? scj : 0.f;
            v[j] = sc[j] != 0.f ? *(const float2*)(base + s * stride + 2 * lane) : make_float2(0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            o0 += v[j].x * sc[j];
            o1 += v[j].y * sc[j];
        }
    }
    s_o[pc][wq][2 * lane] = o0;
    s_o[pc][wq][2 * lane + 1] = o1;
    __syncthreads();
    if (wq != 0 || !valid) return;
    o0 = ((s_o[pc][0][2 * lane] + s_o[pc][1][2 * lane]) + s_o[pc][2][2 * lane]) + s_o[pc][3][2 * lane];
    o1 = ((s_o[pc][0][2 * lane + 1] + s_o[pc][1][2 * lane + 1]) + s_o[pc][2][2 * lane + 1]) + s_o[pc][3][2 * lane + 1];
    const float inv = 1.0f / L;
    const float x0 = o0 * inv, x1 = o1 * inv;
    const float ms = warp_sum(x0 * x0 + x1 * x1) * (1.0f / 64.0f);
    const float rstd = 1.0f / sqrtf(ms + 1e-5f);
    const float g0 = __low2float(og2), g1 = __high2float(og2);
    const float s0 = 1.0f / (1.0f + expf(-g0)), s1 = 1.0f / (1.0f + expf(-g1));
    __nv_bfloat162 out = __floats2bfloat162_rn(x0 * rstd * s0, x1 * rstd * s1);
    *(__nv_bfloat162*)(a.x_attn + (size_t)tok * a.qh * kHeadDim + head * kHeadDim + 2 * lane) = out;
    RT(6, 2)
}

static void attn_cfg(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, cudaStream_t stream, bool pdl) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg = cudaLaunchConfig_t{};
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
}

cudaError_t attn_split_launch(const AttnArgs& a, cudaStream_t stream, bool pdl) {
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t cfg;
    attn_cfg(cfg, attr, stream, pdl);
    cfg.gridDim = dim3(a.splits, a.kvh, 1);
    cfg.blockDim = dim3(32 * ((a.R + 15) / 16), 1, 1);
    return cudaLaunchKernelEx(&cfg, attn_split_kernel, a);
}

cudaError_t attn_combine_launch(const AttnArgs& a, cudaStream_t stream, bool pdl) {
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t cfg;
    attn_cfg(cfg, attr, stream, pdl);
    const int pairs = a.M * a.qh;  // two (token, head) pairs per CTA, four warps each
    cfg.gridDim = dim3((pairs + 1) / 2, 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    return cudaLaunchKernelEx(&cfg, attn_combine_kernel, a);
}

}  // namespace mk

RT_READ(mk_attn_trace_read)
