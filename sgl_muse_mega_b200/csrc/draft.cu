// The DFlash2 draft's row kernels: everything between the draft's GEMMs (which run on the item engine of segments.cuh).
//
// Arithmetic follows the reference's test/reference/dflash2.py operation by operation (f32 elementwise steps in its order,
// no fused multiply-add where it has a separate multiply and add, one bf16 rounding where it rounds):
//   rms_norm / add_rms_norm :245-266   head_norm_rope :275-294   grouped_conv :297-316   attention :338-361
//   topk_low_id :391-399   lattice :587-606   selector_walk :609-640   all_reduce :214-222
// Sums of squares are held to about 2^-45 in two f32 words (the reference's mean is an f64 mean rounded to f32).
//
// Every kernel waits for its predecessor with griddepcontrol.wait before its first dependent read; exchange waits are
// bounded (params.h). Nothing here traps: an index outside its table is clamped and recorded in the status block (code 4).
#include "draft_rows.cuh"

namespace mk {

namespace {

constexpr int kRowThreads = 256;

// Block-wide sum of two-word sums; `red` holds 33 of them in shared memory.
__device__ __forceinline__ double block_sum_f2(F2 v, F2* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum_f2(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        F2 s = lane < nw ? red[lane] : F2{0.f, 0.f};
        s = warp_sum_f2(s);
        if (lane == 0) red[32] = s;
    }
    __syncthreads();
    return f2_value(red[32]);
}
// ---- captured residuals -> fc's input rows ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(kRowThreads) dfeats_kernel(const DFeatsArgs a) {
    griddep_wait();
    const int row = blockIdx.x / a.n_cap, f = blockIdx.x - row * a.n_cap;
    const float4* src = (const float4*)(a.cap[f] + (size_t)row * a.hidden);
    uint2* dst = (uint2*)(a.feats + ((size_t)row * a.n_cap + f) * a.hidden);
    for (int i = threadIdx.x; i < a.hidden / 4; i += kRowThreads) {
        const float4 v = src[i];
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        dst[i] = make_uint2(*(const unsigned*)&lo, *(const unsigned*)&hi);
    }
}

// ---- norm rows -------------------------------------------------------------------------------------------------------------
// One CTA per row, one thread per 8 consecutive channels (16-byte loads; H / 8 threads). A conv group spans a multiple of 8
// channels, so a thread's channels share their dynamic coefficients.
// The all-reduced values of 8 channels of a row: the ranks' bf16 partials summed in rank order in f32, rounded to bf16.
__device__ __forceinline__ void ar8(const DNormArgs& a, int row, int ch0, float (&x)[8]) {
    load8(a.ar + (size_t)row * a.H + ch0, x);
    for (int r = 1; r < a.ranks; ++r) {
        float p[8];
        load8(a.ar + ((size_t)r * 16 + row) * a.H + ch0, p);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = __fadd_rn(x[i], p[i]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = bf16_round(x[i]);
}

__global__ void __launch_bounds__(1024) dnorm_kernel(const DNormArgs a) {
    __shared__ F2 red[33];
    __shared__ long long s_tok;
    griddep_wait();
    xchg_wait(a.wait);
    const int row = blockIdx.x, tid = threadIdx.x, ch0 = tid * 8;
    const bf16* src = a.x ? a.x + (size_t)row * a.H : nullptr;
    if (a.emb_ranks > 0) {
        if (tid == 0) {
            long long tok = row == 0 ? a.words[kWordAnchor] : a.mask_id;
            const long long vocab = a.shard_rows * a.emb_ranks;
            if (tok < 0 || tok >= vocab) {
                record_clamp(a.status, 400, tok);
                tok = tok < 0 ? 0 : vocab - 1;
            }
            s_tok = tok;
        }
        __syncthreads();
        src = a.embed[s_tok / a.shard_rows] + (size_t)(s_tok % a.shard_rows) * a.H;
    }
    float x[8];
    if (a.ar != nullptr) {
        ar8(a, row, ch0, x);
        if (a.coeff != nullptr) {  // the conv's side 1 over the all-reduced rows; coeff row: [side][tap][group]
            const int g = ch0 / (a.H / a.groups);
            const bf16* c = a.coeff + (size_t)row * 4 * a.groups + 2 * a.groups;
            const float d0 = __bfloat162float(c[g]), d1 = __bfloat162float(c[a.groups + g]);
            float b0[8], b1[8], xp[8];
            load8(a.base + (size_t)2 * a.H + ch0, b0);
            if (row > 0) {
                load8(a.base + (size_t)3 * a.H + ch0, b1);
                ar8(a, row - 1, ch0, xp);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float out = __fmul_rn(__fadd_rn(b0[i], d0), x[i]);
                if (row > 0) out = __fadd_rn(out, __fmul_rn(__fadd_rn(b1[i], d1), xp[i]));
                x[i] = bf16_round(out);
            }
        }
    } else {
        load8(src + ch0, x);
    }
    if (a.x_out != nullptr) store8(a.x_out + (size_t)row * a.H + ch0, x);
    F2 sq = {0.f, 0.f};
    if (a.residual != nullptr) {
        float r[8];
        load8(a.residual + (size_t)row * a.H + ch0, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = __fadd_rn(x[i], r[i]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) f2_add_sq(sq, x[i]);
    const float ms = (float)(block_sum_f2(sq, red) / (double)a.H);
    const float rs = rsqrt_exact(__fadd_rn(ms, a.eps));
    float w[8], h[8];
    load8(a.w + ch0, w);
#pragma unroll
    for (int i = 0; i < 8; ++i) h[i] = __fmul_rn(__fmul_rn(x[i], rs), w[i]);
    store8(a.h + (size_t)row * a.H + ch0, h);
    if (a.res_out != nullptr) store8(a.res_out + (size_t)row * a.H + ch0, x);
}

// ---- grouped conv, side 0 -----------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) dconv_kernel(const DConvArgs a) {
    griddep_wait();
    const int row = blockIdx.x, ch0 = threadIdx.x * 8, g = ch0 / (a.H / a.groups);
    const bf16* c = a.coeff + (size_t)row * 4 * a.groups;  // side 0: taps at [0, groups) and [groups, 2 groups)
    const float d0 = __bfloat162float(c[g]), d1 = __bfloat162float(c[a.groups + g]);
    float b0[8], b1[8], x[8], xp[8], out[8];
    load8(a.base + ch0, b0);
    load8(a.h + (size_t)row * a.H + ch0, x);
    if (row > 0) {
        load8(a.base + a.H + ch0, b1);
        load8(a.h + (size_t)(row - 1) * a.H + ch0, xp);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        out[i] = __fmul_rn(__fadd_rn(b0[i], d0), x[i]);
        if (row > 0) out[i] = __fadd_rn(out[i], __fmul_rn(__fadd_rn(b1[i], d1), xp[i]));
    }
    store8(a.out + (size_t)row * a.H + ch0, out);
}

__global__ void __launch_bounds__(kRowThreads) dqkv_rows_kernel(const DQkvRowsArgs a) {
    griddep_wait();
    const int lane = threadIdx.x & 31, heads = a.qh + 2 * a.kvh;
    const long long P = a.words[kWordP];
    for (int w = blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5); w < a.M * heads; w += gridDim.x * (kRowThreads / 32)) {
        const int m = w / heads, head = w - m * heads;
        const bf16* x = a.qkv + ((size_t)m * heads + head) * kDraftHeadDim;
        const __nv_bfloat162 xl = *(const __nv_bfloat162*)(x + 2 * lane), xh = *(const __nv_bfloat162*)(x + 64 + 2 * lane);
        float v[4] = {__low2float(xl), __high2float(xl), __low2float(xh), __high2float(xh)};
        dqkv_head(a, m, head, v, P, lane);
    }
}

// The context rows of the last commit: row i sits at position P - commit + i; rows >= commit are not written.
__global__ void __launch_bounds__(kRowThreads) dctx_kv_kernel(const DCtxKvArgs a) {
    griddep_wait();
    const int lane = threadIdx.x & 31, per_row = a.layers * 2 * a.kvh;
    const long long P = a.words[kWordP], commit = a.words[kWordCommit];
    for (int w = blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5); w < a.M * per_row; w += gridDim.x * (kRowThreads / 32)) {
        const int m = w / per_row, rest = w - m * per_row, layer = rest / (2 * a.kvh), hv = rest - layer * 2 * a.kvh;
        if (m >= commit) continue;
        const long long p = P - commit + m;
        const long long pos = clamp_pos(p, a.rope_rows, a.status, 420);
        const size_t slot = (size_t)(p % a.pool_rows + a.pool_rows) % a.pool_rows;
        const bf16* x = a.kv + ((size_t)m * per_row + rest) * kDraftHeadDim;
        if (hv < a.kvh) {
            head_norm_rope(x, a.k_norm[layer], a.eps, a.rope + pos * kDraftHeadDim, false,
                           a.k_pool[layer] + (slot * a.kvh + hv) * kDraftHeadDim, lane);
        } else {
            uint2* dst = (uint2*)(a.v_pool[layer] + (slot * a.kvh + (hv - a.kvh)) * kDraftHeadDim);
            dst[lane] = ((const uint2*)x)[lane];
        }
    }
}

// ---- non-causal sliding-window attention, head dim 128 -----------------------------------------------------------------------------
// grid (nsplit, kvh): a CTA scores the M x G query rows of one kv head (at most 128; 16 per warp) against one block of 64
// key positions and leaves (max, sum, unnormalised output) per row; the merge kernel combines the blocks. Tensor cores
// through mma.sync m16n8k16 (bf16, f32 accumulate): S = Q K^T with K row-major as the column operand, then the
// probabilities, rounded to bf16, re-used in registers as the row operand of P V with V transposed in shared memory.
// Rows are padded by 8 elements so that a fragment load's 32 lanes fall into 32 distinct banks.
constexpr int kAQ = 128;  // query rows per kv head (M x G <= 128)
constexpr int kAKeys = kDraftKeysPerSplit;
constexpr int kAQs = 128 + 8, kAVs = kAKeys + 8;  // row strides (elements) of Q / K and of V^T
constexpr size_t kAttnSmem = ((size_t)kAQ * kAQs + (size_t)kAKeys * kAQs + (size_t)128 * kAVs) * 2;

__global__ void __launch_bounds__(256, 1) dattn_split_kernel(const DAttnArgs a) {
    extern __shared__ __align__(16) unsigned char sm_raw[];
    bf16* Qs = (bf16*)sm_raw;           // [128][136]
    bf16* Ks = Qs + kAQ * kAQs;         // [64][136]
    bf16* Vt = Ks + kAKeys * kAQs;      // [128 d][72]
    griddep_wait();
    const int tid = threadIdx.x, split = blockIdx.x, h = blockIdx.y;
    const int G = a.qh / a.kvh, R = a.M * G;
    const long long P = a.words[kWordP];
    const long long lo = P - a.left > 0 ? P - a.left : 0, hi = P + a.M - 1;
    const long long key0 = lo + (long long)split * kAKeys;
    float* wsb = a.ws + ((size_t)h * a.nsplit + split) * R * 132;
    if (key0 > hi) {  // no keys here: an empty partial
        for (int r = tid; r < R; r += 256) {
            wsb[(size_t)r * 132] = -INFINITY;
            wsb[(size_t)r * 132 + 1] = 0.f;
        }
        return;
    }
    // Q rows r = b G + g of this kv head (rows past R are zero), 16 bytes a thread
    for (int i = tid; i < kAQ * 16; i += 256) {
        const int r = i >> 4, c = i & 15;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < R) {
            const int b = r / G, g = r - b * G;
            v = *(const uint4*)(a.q + ((size_t)b * a.qh + h * G + g) * 128 + c * 8);
        }
        *(uint4*)(Qs + r * kAQs + c * 8) = v;
    }
    for (int i = tid; i < kAKeys * 16; i += 256) {
        const int kk = i >> 4, c = i & 15;
        const long long pk = key0 + kk;
        uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
        if (pk <= hi) {
            const size_t slot = (size_t)(pk % a.pool_rows);
            kv = *(const uint4*)(a.k_pool + (slot * a.kvh + h) * 128 + c * 8);
            vv = *(const uint4*)(a.v_pool + (slot * a.kvh + h) * 128 + c * 8);
        }
        *(uint4*)(Ks + kk * kAQs + c * 8) = kv;
        const bf16* ve = (const bf16*)&vv;
#pragma unroll
        for (int e = 0; e < 8; ++e) Vt[(c * 8 + e) * kAVs + kk] = ve[e];
    }
    __syncthreads();
    const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int r0 = warp * 16 + g, r1 = r0 + 8;
    // S = Q K^T: 8 key tiles of 8, 8 steps of 16 over the head dimension
    float sc[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) sc[nt][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        const uint32_t a0 = *(const uint32_t*)(Qs + r0 * kAQs + ks * 16 + 2 * t), a1 = *(const uint32_t*)(Qs + r1 * kAQs + ks * 16 + 2 * t);
        const uint32_t a2 = *(const uint32_t*)(Qs + r0 * kAQs + ks * 16 + 8 + 2 * t), a3 = *(const uint32_t*)(Qs + r1 * kAQs + ks * 16 + 8 + 2 * t);
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const uint32_t b0 = *(const uint32_t*)(Ks + (nt * 8 + g) * kAQs + ks * 16 + 2 * t);
            const uint32_t b1 = *(const uint32_t*)(Ks + (nt * 8 + g) * kAQs + ks * 16 + 8 + 2 * t);
            mma_bf16_16816(sc[nt], a0, a1, a2, a3, b0, b1);
        }
    }
    // mask, row max, probabilities (a row's 64 scores sit in the 4 lanes of its quad)
    const float scale = 0.08838834764831845f;  // 128^-0.5
    const long long pq0 = P + r0 / G, pq1 = P + r1 / G;
    float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const long long pk = key0 + nt * 8 + 2 * t + (i & 1);
            const bool top = i < 2;
            const long long pq = top ? pq0 : pq1;
            const bool seen = (top ? r0 : r1) < R && pk <= hi && pk >= pq - a.left && pk <= pq + a.left;
            const float v = seen ? sc[nt][i] * scale : -INFINITY;
            sc[nt][i] = v;
            if (top) m0 = fmaxf(m0, v);
            else m1 = fmaxf(m1, v);
        }
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 1));
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 2));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 1));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 2));
    float l0 = 0.f, l1 = 0.f;
    uint32_t pa[8][2];  // probabilities as bf16 pairs: [key tile][row r0 | row r1]
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        const float p0 = m0 == -INFINITY ? 0.f : expf(sc[nt][0] - m0), p1 = m0 == -INFINITY ? 0.f : expf(sc[nt][1] - m0);
        const float p2 = m1 == -INFINITY ? 0.f : expf(sc[nt][2] - m1), p3 = m1 == -INFINITY ? 0.f : expf(sc[nt][3] - m1);
        const __nv_bfloat162 q0 = __floats2bfloat162_rn(p0, p1), q1 = __floats2bfloat162_rn(p2, p3);
        // the sums run over the rounded probabilities, the values the output is built from
        l0 += __low2float(q0) + __high2float(q0);
        l1 += __low2float(q1) + __high2float(q1);
        pa[nt][0] = *(const uint32_t*)&q0;
        pa[nt][1] = *(const uint32_t*)&q1;
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    // O = P V: 4 steps of 16 keys, 16 tiles of 8 over the head dimension, in two halves to bound the registers
    float* o0 = wsb + (size_t)r0 * 132;
    float* o1 = wsb + (size_t)r1 * 132;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        float oc[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) oc[nt][i] = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const int d = (half * 8 + nt) * 8 + g;
                const uint32_t b0 = *(const uint32_t*)(Vt + d * kAVs + j * 16 + 2 * t), b1 = *(const uint32_t*)(Vt + d * kAVs + j * 16 + 8 + 2 * t);
                mma_bf16_16816(oc[nt], pa[2 * j][0], pa[2 * j][1], pa[2 * j + 1][0], pa[2 * j + 1][1], b0, b1);
            }
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int d = (half * 8 + nt) * 8 + 2 * t;
            if (r0 < R) *(float2*)(o0 + 4 + d) = make_float2(oc[nt][0], oc[nt][1]);
            if (r1 < R) *(float2*)(o1 + 4 + d) = make_float2(oc[nt][2], oc[nt][3]);
        }
    }
    if (t == 0) {
        if (r0 < R) {
            o0[0] = m0;
            o0[1] = l0;
        }
        if (r1 < R) {
            o1[0] = m1;
            o1[1] = l1;
        }
    }
}

// One warp per (window row, q head): the blocks' partials combined in block order. The blocks' (max, sum) pairs are read
// lane-parallel (two blocks a lane, at most 64 blocks), the rescaled outputs accumulated with the loads of several blocks
// in flight.
__global__ void __launch_bounds__(kRowThreads) dattn_merge_kernel(const DAttnArgs a) {
    griddep_wait();
    const int lane = threadIdx.x & 31, G = a.qh / a.kvh, R = a.M * G;
    for (int w = blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5); w < a.M * a.qh; w += gridDim.x * (kRowThreads / 32)) {
        const int b = w / a.qh, head = w - b * a.qh, h = head / G, r = b * G + (head - h * G);
        const float* base = a.ws + ((size_t)h * a.nsplit * R + r) * 132;
        const size_t stride = (size_t)R * 132;
        const float ma = lane < a.nsplit ? base[lane * stride] : -INFINITY, mb = lane + 32 < a.nsplit ? base[(lane + 32) * stride] : -INFINITY;
        const float la = lane < a.nsplit ? base[lane * stride + 1] : 0.f, lb = lane + 32 < a.nsplit ? base[(lane + 32) * stride + 1] : 0.f;
        const float mx = warp_max(fmaxf(ma, mb));
        const float fa = ma == -INFINITY ? 0.f : expf(ma - mx), fb = mb == -INFINITY ? 0.f : expf(mb - mx);
        const float l = warp_sum(la * fa + lb * fb);
        float o[4] = {0.f, 0.f, 0.f, 0.f};
        // eight blocks' rows are requested before the first is used: the loop is one L2 round trip per eight blocks
        for (int s0 = 0; s0 < a.nsplit; s0 += 8) {
            float2 v0[8], v1[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float* p = base + (size_t)min(s0 + j, a.nsplit - 1) * stride;
                v0[j] = *(const float2*)(p + 4 + 2 * lane);
                v1[j] = *(const float2*)(p + 4 + 64 + 2 * lane);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int s = s0 + j;
                float f = __shfl_sync(0xffffffffu, s < 32 ? fa : fb, s & 31);
                if (s >= a.nsplit) f = 0.f;
                // an empty block has f = 0 and output words that were never written: select, do not multiply
                o[0] += f == 0.f ? 0.f : v0[j].x * f;
                o[1] += f == 0.f ? 0.f : v0[j].y * f;
                o[2] += f == 0.f ? 0.f : v1[j].x * f;
                o[3] += f == 0.f ? 0.f : v1[j].y * f;
            }
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
        bf16* out = a.o + ((size_t)b * a.qh + head) * 128;
        *(__nv_bfloat162*)(out + 2 * lane) = __floats2bfloat162_rn(o[0] * inv, o[1] * inv);
        *(__nv_bfloat162*)(out + 64 + 2 * lane) = __floats2bfloat162_rn(o[2] * inv, o[3] * inv);
    }
}

// ---- candidates: top-16 by (value descending, id ascending) -------------------------------------------------------------------------
// A key orders both at once: the bf16-rounded logit as a sortable 32-bit pattern above the complemented id.
__device__ __forceinline__ unsigned long long topk_key(float logit, unsigned id) {
    unsigned u = __float_as_uint(bf16_round(logit));
    if (logit != logit) u = 0xFFFFFFFFu;  // NaN sorts above every number, as torch's descending sort places it
    else u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - id);
}
__device__ __forceinline__ float key_value(unsigned long long k) {
    unsigned u = (unsigned)(k >> 32);
    if (u == 0xFFFFFFFFu) return __uint_as_float(0x7FC00000u);
    u = (u & 0x80000000u) ? (u & 0x7FFFFFFFu) : ~u;
    return __uint_as_float(u);
}
__device__ __forceinline__ unsigned key_id(unsigned long long k) { return 0xFFFFFFFFu - (unsigned)(k & 0xFFFFFFFFull); }

// The 16 largest of the block's register-held keys (PER per thread; 0 = empty) -> out[0..16), descending. Each warp
// selects its own 16 with shuffles only, then warp 0 selects among the 8 x 16 survivors: two block barriers in all.
// `wl` holds 128 keys of shared memory.
template <int PER, typename KEY>
__device__ __forceinline__ void block_top16(KEY (&k)[PER], KEY* out, KEY* wl) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int round = 0; round < kDraftTopK; ++round) {
        KEY best = 0;
#pragma unroll
        for (int j = 0; j < PER; ++j) best = k[j] > best ? k[j] : best;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const KEY other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        if (best != 0) {
#pragma unroll
            for (int j = 0; j < PER; ++j)
                if (k[j] == best) k[j] = 0;
        }
        if (lane == 0) wl[warp * kDraftTopK + round] = best;
    }
    __syncthreads();
    if (warp == 0) {
        KEY m[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) m[j] = wl[lane + 32 * j];
        for (int round = 0; round < kDraftTopK; ++round) {
            KEY best = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) best = m[j] > best ? m[j] : best;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const KEY other = __shfl_xor_sync(0xffffffffu, best, o);
                best = other > best ? other : best;
            }
            if (best != 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (m[j] == best) m[j] = 0;
            }
            if (lane == 0) out[round] = best;
        }
    }
    __syncthreads();
}

// Inside a chunk of 4096 ids a 32-bit key orders (value descending, id ascending): the bf16 value as a sortable 16-bit
// pattern above the complemented 12-bit position; the selection then runs on single registers.
__device__ __forceinline__ unsigned chunk_key(float logit, unsigned pos) {
    unsigned h = __float_as_uint(bf16_round(logit)) >> 16;
    if (logit != logit) h = 0xFFFFu;  // NaN sorts above every number
    else h = (h & 0x8000u) ? (~h & 0xFFFFu) : (h | 0x8000u);
    return (h << 12) | (4095u - pos);
}
__device__ __forceinline__ unsigned long long chunk_key_global(unsigned k, unsigned chunk) {
    if (k == 0) return 0ull;
    const unsigned h = k >> 12, pos = 4095u - (k & 4095u);
    // the 32-bit pattern topk_key makes of the same value (its low 16 bits are zeros, complemented for negatives)
    const unsigned u = h == 0xFFFFu ? 0xFFFFFFFFu : (h & 0x8000u) ? (h << 16) : ((h << 16) | 0xFFFFu);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (chunk * (unsigned)kDraftTopkChunk + pos));
}

constexpr int kMaxMergePer = kMaxMergeChunks * kDraftTopK / kRowThreads;

// grid (chunks, rows): every CTA leaves its chunk's 16 best; the last CTA of a row to finish merges the row's lists into
// the row's slot `nchunk` of the key buffer (the 16 candidates, descending).
__global__ void __launch_bounds__(kRowThreads) dtopk_kernel(const DTopkArgs a) {
    __shared__ unsigned long long red[(kRowThreads / 32) * kDraftTopK];
    __shared__ unsigned s_win[kDraftTopK];
    __shared__ unsigned s_last;
    griddep_wait();
    xchg_wait(a.wait);
    const int chunk = blockIdx.x, row = blockIdx.y;
    constexpr int PER = kDraftTopkChunk / kRowThreads;
    unsigned k[PER];
    const long long start = (long long)chunk * kDraftTopkChunk;
    const float* src = a.logits + (size_t)row * a.V;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const unsigned pos = threadIdx.x + j * kRowThreads;
        k[j] = start + pos < a.V ? chunk_key(src[start + pos], pos) : 0u;
    }
    block_top16<PER, unsigned>(k, s_win, (unsigned*)red);
    unsigned long long* row_keys = a.keys + (size_t)row * (a.nchunk + 1) * kDraftTopK;
    if (threadIdx.x < kDraftTopK) row_keys[chunk * kDraftTopK + threadIdx.x] = chunk_key_global(s_win[threadIdx.x], (unsigned)chunk);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(a.row_count + row, 1u) == (unsigned)a.nchunk - 1 ? 1u : 0u;
    __syncthreads();
    if (s_last == 0) return;
    __threadfence();
    if (threadIdx.x == 0) a.row_count[row] = 0;
    unsigned long long m[kMaxMergePer];
    const int n = a.nchunk * kDraftTopK;
#pragma unroll
    for (int j = 0; j < kMaxMergePer; ++j) {
        const int i = threadIdx.x + j * kRowThreads;
        m[j] = i < n ? __ldcg(row_keys + i) : 0ull;
    }
    block_top16<kMaxMergePer, unsigned long long>(m, row_keys + (size_t)a.nchunk * kDraftTopK, red);
}

// ---- lattice and walk ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kRowThreads) dlattice_kernel(const DLatticeArgs a) {
    __shared__ unsigned long long s_cur[kDraftTopK], s_prev[kDraftTopK];
    __shared__ float s_hid[512];
    __shared__ __align__(16) unsigned s_A[kDraftTopK][257];  // codebook rows as bf16 pairs, padded against bank conflicts
    __shared__ __align__(16) unsigned s_S[kDraftTopK][257];
    __shared__ long long s_pred[kDraftTopK];
    __shared__ float s_unary[kDraftTopK];
    __shared__ unsigned s_last;
    griddep_wait();
    const int e = blockIdx.x, tid = threadIdx.x;
    // the rows' 16 candidates, merged by the top-k kernel (slot nchunk of a row's key lists)
    if (tid < kDraftTopK) {
        s_cur[tid] = a.keys[((size_t)e * (a.nchunk + 1) + a.nchunk) * kDraftTopK + tid];
        if (e > 0) s_prev[tid] = a.keys[((size_t)(e - 1) * (a.nchunk + 1) + a.nchunk) * kDraftTopK + tid];
    }
    __syncthreads();
    for (int i = tid; i < a.R; i += kRowThreads) s_hid[i] = __bfloat162float(a.hid[(size_t)e * a.R + i]);
    if (tid < kDraftTopK) {
        const float v = key_value(s_cur[tid]);
        const float u = __fmul_rn(tanhf(__fdiv_rn(__fmul_rn(v, a.mult), a.cap)), a.cap);
        s_unary[tid] = u;
        a.cand[(size_t)e * kDraftTopK + tid] = (long long)key_id(s_cur[tid]);
        a.unary[(size_t)e * kDraftTopK + tid] = u;
    }
    __syncthreads();
    if (tid < kDraftTopK) {
        long long pred = e == 0 ? a.words[kWordAnchor] : (long long)key_id(s_prev[tid]);
        if (pred < 0 || pred >= a.vocab) {
            record_clamp(a.status, 430, pred);
            pred = pred < 0 ? 0 : a.vocab - 1;
        }
        s_pred[tid] = pred;
    }
    __syncthreads();
    {  // the 16 predecessor rows of A and the 16 candidate rows of S, coalesced
        const int words = a.R / 2;
        for (int i = tid; i < kDraftTopK * words; i += kRowThreads) {
            const int r = i / words, w = i - r * words;
            s_A[r][w] = ((const unsigned*)(a.pred + (size_t)s_pred[r] * a.R))[w];
            s_S[r][w] = ((const unsigned*)(a.succ + (size_t)key_id(s_cur[r]) * a.R))[w];
        }
    }
    __syncthreads();
    {
        const int p = tid >> 4, c = tid & 15;
        // The reference sums the products in f64 and rounds once to bf16. Every product of two bf16 values is exact in f32;
        // the sum runs in f32 with the rounding error of each addition captured exactly (two-sum) and carried in a second
        // word, so the pair holds the sum to about 2^-46: f64 arithmetic is scarce on this part and made this kernel 17 us
        // longer.
        float hi = 0.f, lo = 0.f;
        auto add = [&](float x) {
            const float t = __fadd_rn(hi, x), bb = __fsub_rn(t, hi);
            lo = __fadd_rn(lo, __fadd_rn(__fsub_rn(hi, __fsub_rn(t, bb)), __fsub_rn(x, bb)));
            hi = t;
        };
        for (int w = 0; w < a.R / 2; ++w) {
            const unsigned au = s_A[p][w], su = s_S[c][w];
            const __nv_bfloat162 av = *(const __nv_bfloat162*)&au, sv = *(const __nv_bfloat162*)&su;
            // the product A x hid is exact in f32 (two bf16 factors) and rounded to bf16 as the reference stores it
            const float p0 = bf16_round(__fmul_rn(__low2float(av), s_hid[2 * w])), p1 = bf16_round(__fmul_rn(__high2float(av), s_hid[2 * w + 1]));
            add(__fmul_rn(p0, __low2float(sv)));
            add(__fmul_rn(p1, __high2float(sv)));
        }
        a.scores[((size_t)e * kDraftTopK + p) * kDraftTopK + c] =
            __fadd_rn(s_unary[c], __bfloat162float(__double2bfloat16((double)hi + (double)lo)));
    }
    // the last block to finish walks the lattice
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(a.counter, 1u) == gridDim.x - 1 ? 1u : 0u;
    __syncthreads();
    if (s_last == 0) return;
    __threadfence();
    // the whole lattice (gamma x 16 x 16 scores, 15 KB) and the candidates into shared memory, then one thread walks it
    float* s_sc = (float*)&s_A[0][0];             // 16 x 257 words hold gamma x 256 scores (gamma <= 15)
    long long* s_cd = (long long*)&s_S[0][0];     // gamma x 16 candidates
    for (int i = tid; i < a.gamma * kDraftTopK * kDraftTopK; i += kRowThreads) s_sc[i] = __ldcg(a.scores + i);
    for (int i = tid; i < a.gamma * kDraftTopK; i += kRowThreads) s_cd[i] = __ldcg(a.cand + i);
    __syncthreads();
    if (tid == 0) {
        *a.counter = 0;
        int prev = 0;
        a.verify_ids[0] = a.words[kWordAnchor];
        for (int s = 0; s < a.gamma; ++s) {
            const float* row = s_sc + (s * kDraftTopK + prev) * kDraftTopK;
            int idx = -1;
            if (a.samp != nullptr) {
                // sampled: q = softmax(row / T) in f32 (T clamped at 1e-5), index = #{c : u >= cumsum(q)_c} clamped to 15;
                // u = the top 24 bits of word s % 4 of Philox4x32-10({iteration, stream, purpose 0, s / 4}, seed)
                const float T = fmaxf(__uint_as_float((unsigned)((unsigned long long)a.samp[3] & 0xFFFFFFFFull)), 1e-5f);
                float sc[kDraftTopK], mx = -INFINITY, sum = 0.f;
                for (int c = 0; c < kDraftTopK; ++c) {
                    sc[c] = __fdiv_rn(row[c], T);
                    mx = fmaxf(mx, sc[c]);
                }
                for (int c = 0; c < kDraftTopK; ++c) {
                    sc[c] = expf(__fsub_rn(sc[c], mx));
                    sum = __fadd_rn(sum, sc[c]);
                }
                const unsigned long long seed = (unsigned long long)a.samp[0];
                const uint4 r4 = philox4x32(make_uint4((unsigned)a.words[kWordIter], (unsigned)a.samp[1], 0u, (unsigned)s / 4),
                                            make_uint2((unsigned)seed, (unsigned)(seed >> 32)));
                const unsigned rw[4] = {r4.x, r4.y, r4.z, r4.w};
                const float u = (float)(rw[s & 3] >> 8) * 0x1p-24f;
                float cum = 0.f;
                idx = 0;
                for (int c = 0; c < kDraftTopK; ++c) {
                    const float q = __fdiv_rn(sc[c], sum);
                    cum = __fadd_rn(cum, q);
                    idx += u >= cum;
                    if (a.walk_q != nullptr) a.walk_q[s * kDraftTopK + c] = q;
                }
                idx = min(idx, kDraftTopK - 1);
            }
            for (int c = 0; a.samp == nullptr && c < kDraftTopK && idx < 0; ++c)
                if (row[c] != row[c]) idx = c;  // the first NaN wins
            if (idx < 0) {
                idx = 0;
                float best = row[0];
                for (int c = 1; c < kDraftTopK; ++c)
                    if (row[c] > best) {
                        best = row[c];
                        idx = c;
                    }
            }
            const long long tok = s_cd[s * kDraftTopK + idx];
            a.drafts[s] = tok;
            a.verify_ids[1 + s] = tok;
            a.pick[s] = idx;
            prev = idx;
        }
    }
}

// ---- the draft's rings -> the serving pool ---------------------------------------------------------------------------------------------
// state[0]: the position up to which the pool holds the request's context; state[1 + i]: the pool slot of position
// state[0] + i (the window slots of the iteration that committed them). lag 1 (an iteration's last launch): the rings
// hold the positions below P - commit; lag 0 (after a draft that ran alone): below P. One CTA.
__global__ void __launch_bounds__(kRowThreads) dkv_sync_kernel(const DKvSyncArgs a) {
    __shared__ long long s_slot[16];
    __shared__ long long s_from;
    __shared__ int s_n;
    griddep_wait();
    const int t = threadIdx.x;
    if (t == 0) {
        const long long from = a.state[0], to = a.words[kWordP] - (a.lag ? a.words[kWordCommit] : 0);
        long long n = to - from;
        if (n < 0 || n > 16) {  // the pool and the rings disagree: copy nothing, say so
            record_clamp(a.status, 440, n);
            n = 0;
        }
        s_from = from;
        s_n = (int)n;
    }
    if (t < 16) s_slot[t] = a.state[1 + t];
    __syncthreads();
    const long long from = s_from;
    const int n = s_n, q = a.row_bytes / 16;
    for (int i = t; i < a.n_buf * n * q; i += kRowThreads) {
        const int k = i % q, r = i / q % n, b = i / (q * n);
        const long long ring_row = ((from + r) % a.ring_rows + a.ring_rows) % a.ring_rows;
        const uint4* src = (const uint4*)a.ring[b] + (size_t)ring_row * q + k;
        ((uint4*)a.pool[b])[(size_t)s_slot[r] * q + k] = *src;
    }
    __syncthreads();
    if (t == 0) a.state[0] = from + n;
    if (a.lag && t < 16) a.state[1 + t] = a.window[t];
}

template <typename Args>
cudaError_t launch_d(void (*kern)(const Args), dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool pdl, const Args& a) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, a);
}

}  // namespace

size_t dattn_smem() { return kAttnSmem; }

cudaError_t draft_prepare() {
    return cudaFuncSetAttribute(dattn_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAttnSmem);
}

cudaError_t dfeats_launch(const DFeatsArgs& a, cudaStream_t s, bool pdl) {
    return launch_d(dfeats_kernel, dim3(a.rows * a.n_cap), dim3(kRowThreads), 0, s, pdl, a);
}
cudaError_t dnorm_launch(const DNormArgs& a, cudaStream_t s, bool pdl) {
    return launch_d(dnorm_kernel, dim3(a.M), dim3(a.H / 8), 0, s, pdl, a);
}
cudaError_t dconv_launch(const DConvArgs& a, cudaStream_t s, bool pdl) {
    return launch_d(dconv_kernel, dim3(a.M), dim3(a.H / 8), 0, s, pdl, a);
}
cudaError_t dqkv_rows_launch(const DQkvRowsArgs& a, cudaStream_t s, bool pdl) {
    const int warps = a.M * (a.qh + 2 * a.kvh);
    return launch_d(dqkv_rows_kernel, dim3((warps + 7) / 8), dim3(kRowThreads), 0, s, pdl, a);
}
cudaError_t dctx_kv_launch(const DCtxKvArgs& a, cudaStream_t s, bool pdl) {
    const int warps = a.M * a.layers * 2 * a.kvh;
    return launch_d(dctx_kv_kernel, dim3((warps + 7) / 8), dim3(kRowThreads), 0, s, pdl, a);
}
cudaError_t dattn_split_launch(const DAttnArgs& a, cudaStream_t s, bool pdl) {
    return launch_d(dattn_split_kernel, dim3(a.nsplit, a.kvh), dim3(256), kAttnSmem, s, pdl, a);
}
cudaError_t dattn_merge_launch(const DAttnArgs& a, cudaStream_t s, bool pdl) {
    return launch_d(dattn_merge_kernel, dim3((a.M * a.qh + 7) / 8), dim3(kRowThreads), 0, s, pdl, a);
}
cudaError_t dtopk_launch(const DTopkArgs& a, cudaStream_t s, bool pdl) {
    return launch_d(dtopk_kernel, dim3(a.nchunk, a.gamma), dim3(kRowThreads), 0, s, pdl, a);
}
cudaError_t dlattice_launch(const DLatticeArgs& a, cudaStream_t s, bool pdl) {
    return launch_d(dlattice_kernel, dim3(a.gamma), dim3(kRowThreads), 0, s, pdl, a);
}
cudaError_t dkv_sync_launch(const DKvSyncArgs& a, cudaStream_t s, bool pdl) {
    return launch_d(dkv_sync_kernel, dim3(1), dim3(kRowThreads), 0, s, pdl, a);
}

}  // namespace mk
