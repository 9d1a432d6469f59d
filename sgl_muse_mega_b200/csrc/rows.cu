// Row kernels of the layer: everything that is not a weight stream. Each works on the window's <= 16 rows in f32 with
// the bf16 rounding points of the reference's contract (test/reference/muse_spark.py:335-435,587-635).
#include "stages.h"

namespace mk {

static __device__ __forceinline__ float inv_sqrt(float x) { return 1.0f / sqrtf(x); }

// ---- all-reduce consume + post norm + gated residual + pre norm ------------------------------------------------------
// mode 0 (post-attention): branch = bf16(sum over ranks of the bf16 partials, rank order, f32); v = branch
// mode 1 (cross-layer):    v = gathered unpooler row x post_w
// stream' = fma(alpha, stream, scaled), normed = bf16((stream' rstd) pre_w)       (muse_spark.py:335-357)

constexpr int kNormThreads = 1024;
constexpr int kNormPer = 8;  // H <= 8192

__global__ void __launch_bounds__(kNormThreads) resid_norm_kernel(const NormArgs a) {
    __shared__ float red[33];
    griddep_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    float v[kNormPer];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kNormPer; ++i) {
        const int c = tid + i * kNormThreads;
        v[i] = 0.f;
        if (c < a.H) {
            if (a.mode == 0) {
                float acc = __bfloat162float(a.src[(size_t)row * a.H + c]);
                for (int r = 1; r < a.ranks; ++r) acc += __bfloat162float(a.src[((size_t)r * a.M + row) * a.H + c]);
                const bf16 b = __float2bfloat16_rn(acc);
                a.branch[(size_t)row * a.H + c] = b;
                v[i] = __bfloat162float(b);
            } else {
                v[i] = __bfloat162float(a.src[(size_t)row * a.H + c]) * __bfloat162float(a.post_w[c]);
            }
            ss += v[i] * v[i];
        }
    }
    const float post_rstd = inv_sqrt(block_sum(ss, red) / (float)a.H + 1e-8f);
    float ns[kNormPer];
    ss = 0.f;
#pragma unroll
    for (int i = 0; i < kNormPer; ++i) {
        const int c = tid + i * kNormThreads;
        ns[i] = 0.f;
        if (c < a.H) {
            const float beta = a.beta[c];
            const float scaled = a.mode == 0 ? (beta * post_rstd) * v[i] : beta * (v[i] * post_rstd);
            ns[i] = fmaf(a.alpha[c], a.stream_in[(size_t)row * a.H + c], scaled);
            ss += ns[i] * ns[i];
        }
    }
    const float pre_rstd = inv_sqrt(block_sum(ss, red) / (float)a.H + 1e-5f);
#pragma unroll
    for (int i = 0; i < kNormPer; ++i) {
        const int c = tid + i * kNormThreads;
        if (c < a.H) {
            a.stream_out[(size_t)row * a.H + c] = ns[i];
            const bf16 h = __float2bfloat16_rn((ns[i] * pre_rstd) * __bfloat162float(a.pre_w[c]));
            a.normed[(size_t)row * a.H + c] = h;
            if (a.normed_f32) a.normed_f32[(size_t)row * a.H + c] = __bfloat162float(h);
        }
    }
}

// ---- top-k routing -----------------------------------------------------------------------------------------------------
// One warp per row: s = sigmoid(mult x logit) (f64, rounded to f32), sel = s + bias, k rounds of arg-max with the smaller
// id winning ties, weights = ((sel - bias) / (sum in selection order + 1e-15)) x route_scale   (muse_spark.py:378-404)

constexpr int kTopkPer = 32;  // E <= 1024

__global__ void __launch_bounds__(32) topk_kernel(const TopkArgs a) {
    griddep_wait();
    const int row = blockIdx.x, lane = threadIdx.x;
    float sel[kTopkPer];
#pragma unroll
    for (int i = 0; i < kTopkPer; ++i) {
        const int e = lane + 32 * i;
        sel[i] = -INFINITY;
        if (e < a.E) {
            const double z = (double)a.logits[(size_t)row * a.E + e] * a.mult;
            const float s = (float)(1.0 / (1.0 + exp(-z)));
            sel[i] = s + a.bias[e];
        }
    }
    float total = 0.f;
    float mine = 0.f;  // lane j keeps the j-th selected (sel - bias)
    int myid = 0;
    for (int j = 0; j < a.k; ++j) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kTopkPer; ++i) {
            const int e = lane + 32 * i;
            if (sel[i] > bv) { bv = sel[i]; bi = e; }  // ascending e per lane: strict > keeps the smaller id
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        const float sv = bv - a.bias[bi];
        total += sv;
        if (lane == j) { mine = sv; myid = bi; }
        if ((bi & 31) == lane) {
#pragma unroll
            for (int i = 0; i < kTopkPer; ++i)
                if (i == (bi >> 5)) sel[i] = -INFINITY;
        }
    }
    const float inv = 1.0f / (total + 1e-15f);
    if (lane < a.k) {
        a.ids[(size_t)row * a.k + lane] = myid;
        a.w[(size_t)row * a.k + lane] = (mine * inv) * a.route_scale;
    }
}

// ---- pre-expert norm + dynamic NVFP4 quantisation ---------------------------------------------------------------------
// n = bf16(bf16(x rsqrt(mean x^2 + eps)) gamma); NVFP4: x_scale = max(amax, 1e-10) / 2688, per 16:
// sf = e4m3(max(gamax, 1e-10) / 6 / x_scale), code = e2m1(n / max(sf x_scale, 1e-10))           (muse_spark.py:407-435)

__global__ void __launch_bounds__(256) nq_kernel(const NqArgs a) {
    __shared__ float red[33];
    griddep_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    const int groups = a.P / 16;
    const bf16* x = a.pooled + (size_t)row * a.P;
    float ss = 0.f;
    for (int gi = tid; gi < groups; gi += 256) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float v = __bfloat162float(x[gi * 16 + i]);
            ss += v * v;
        }
    }
    const float rstd = inv_sqrt(block_sum(ss, red) / (float)a.P + a.eps);
    float amax = 0.f;
    for (int gi = tid; gi < groups; gi += 256) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float v = __bfloat162float(x[gi * 16 + i]);
            const float n = bf16_round(bf16_round(v * rstd) * __bfloat162float(a.gamma[gi * 16 + i]));
            amax = fmaxf(amax, fabsf(n));
        }
    }
    amax = block_max(amax, red);
    const float kSixth = 1.0f / 6.0f, kInv2688 = 1.0f / 2688.0f;
    const float x_scale = fmaxf(amax, 1e-10f) * kInv2688;
    const float inv_x = 1.0f / x_scale;
    if (tid == 0 && !a.bf16_out) a.x_scale[row] = x_scale;
    for (int gi = tid; gi < groups; gi += 256) {
        float n[16];
        float gmax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float v = __bfloat162float(x[gi * 16 + i]);
            n[i] = bf16_round(bf16_round(v * rstd) * __bfloat162float(a.gamma[gi * 16 + i]));
            gmax = fmaxf(gmax, fabsf(n[i]));
        }
        if (a.bf16_out) {
            bf16* o = (bf16*)a.q + (size_t)row * a.P + gi * 16;
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float2bfloat16_rn(n[i]);
            continue;
        }
        const uint32_t sfb = float_to_e4m3((fmaxf(gmax, 1e-10f) * kSixth) * inv_x);
        const float out_scale = 1.0f / fmaxf(e4m3_to_float(sfb) * x_scale, 1e-10f);
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            lo |= float_to_e2m1(n[i] * out_scale) << (4 * i);
            hi |= float_to_e2m1(n[8 + i] * out_scale) << (4 * i);
        }
        *(uint2*)(a.q + (size_t)row * (a.P / 2) + gi * 8) = make_uint2(lo, hi);
        a.sf[(size_t)row * groups + gi] = (unsigned char)sfb;
    }
}

// ---- route tables (the front) -------------------------------------------------------------------------------------------
// Slots of the live rows grouped by expert: active experts ascending, slots of one expert in slot order.
__global__ void __launch_bounds__(128) route_tables_kernel(const int* ids, int E, int k, int b_live, RouteTables* rt) {
    __shared__ int cnt[1024];
    __shared__ int first[1024];
    griddep_wait();
    const int tid = threadIdx.x, S = b_live * k;
    for (int e = tid; e < E; e += 128) cnt[e] = 0;
    __syncthreads();
    int my_e = -1;
    if (tid < S) {
        my_e = ids[tid];
        atomicAdd(&cnt[my_e], 1);
    }
    __syncthreads();
    if (tid == 0) {
        int na = 0, off = 0;
        for (int e = 0; e < E; ++e) {
            first[e] = off;
            if (cnt[e] > 0) {
                rt->act_e[na] = e;
                rt->act_off[na] = off;
                ++na;
                off += cnt[e];
            }
        }
        rt->act_off[na] = off;
        rt->n_active = na;
    }
    __syncthreads();
    if (tid < S) {
        int before = 0;
        for (int s = 0; s < tid; ++s) before += (ids[s] == my_e);
        rt->slot[first[my_e] + before] = tid;
    }
}

// ---- h row view: scales moved to the row's largest exponent ---------------------------------------------------------------
// e_row = max over the full row's group exponents; sf' = sf x 2^-(e_row - e): exponent-field move while normal, round half
// up on the subnormal grid                                                                 (muse_spark.py:447-491)
__device__ __forceinline__ uint32_t scale_down_byte(uint32_t byte, int delta) {
    const int ef = (int)(byte >> 3);
    if (ef > delta) return byte - ((uint32_t)delta << 3);
    const uint32_t sig = (byte & 7u) | (ef != 0 ? 8u : 0u);
    int sh = delta - ef + (ef != 0 ? 1 : 0);
    sh = min(max(sh, 0), 8);
    const uint32_t half = sh > 0 ? (1u << (sh - 1)) : 0u;
    return (sig + half) >> sh;
}

__global__ void __launch_bounds__(256) hrow_kernel(const unsigned char* z_sf, const signed char* z_ex, int groups, int slots_live,
                                                   unsigned char* z_sfd, float* rowscale) {
    __shared__ float red[33];
    griddep_wait();
    const int slot = blockIdx.x, tid = threadIdx.x;
    if (slot >= slots_live) return;
    float mx = -1000.f;
    for (int gi = tid; gi < groups; gi += 256) mx = fmaxf(mx, (float)z_ex[(size_t)slot * groups + gi]);
    const int e_row = (int)block_max(mx, red);
    for (int gi = tid; gi < groups; gi += 256) {
        const size_t i = (size_t)slot * groups + gi;
        z_sfd[i] = (unsigned char)scale_down_byte(z_sf[i], e_row - (int)z_ex[i]);
    }
    if (tid == 0) rowscale[slot] = __uint_as_float((uint32_t)(e_row + 127) << 23);
}

// ---- per-slot post norm + weighted combine ---------------------------------------------------------------------------------
// xg = zb (gamma + 1); inv = 1 / sqrt(mean xg^2 + 1e-8); y = bf16(sum_j fma(w_j inv_j, xg_j, acc)), j ascending; rows past
// b_live give 0                                                                             (muse_spark.py:587-598)

__global__ void __launch_bounds__(256) combine_kernel(const CombineArgs a) {
    __shared__ float red[33];
    __shared__ float sc[32];
    griddep_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    if (row >= a.b_live) {
        for (int c = tid; c < a.P; c += 256) a.y[(size_t)row * a.P + c] = __float2bfloat16_rn(0.f);
        return;
    }
    for (int j = 0; j < a.k; ++j) {
        const bf16* z = a.zb + ((size_t)row * a.k + j) * a.P;
        float ss = 0.f;
        for (int c = tid; c < a.P; c += 256) {
            const float xg = __bfloat162float(z[c]) * __bfloat162float(a.gamma_p1[c]);
            ss += xg * xg;
        }
        const float ms = block_sum(ss, red) / (float)a.P;
        if (tid == 0) sc[j] = a.w[(size_t)row * a.k + j] * (1.0f / sqrtf(ms + 1e-8f));
    }
    __syncthreads();
    for (int c = tid; c < a.P; c += 256) {
        const float gp = __bfloat162float(a.gamma_p1[c]);
        float acc = 0.f;
        for (int j = 0; j < a.k; ++j) {
            const float xg = __bfloat162float(a.zb[((size_t)row * a.k + j) * a.P + c]) * gp;
            acc = fmaf(sc[j], xg, acc);
        }
        a.y[(size_t)row * a.P + c] = __float2bfloat16_rn(acc);
    }
}

// ---- qkv row ops: qk norm, q scale, interleaved-pair RoPE, KV append -----------------------------------------------------------
// One warp per (row, head) over the q, k and v heads of the bf16 qkv row                    (muse_spark.py:601-635)

__global__ void __launch_bounds__(256) rowops_kernel(const RowopsArgs a) {
    griddep_wait();
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int heads = a.qh + 2 * a.kvh;
    if (w >= a.M * heads) return;
    const int tok = w / heads, head = w % heads;
    bf16* p = a.qkv + (size_t)tok * a.qkv_row + head * kHeadDim + 2 * lane;
    __nv_bfloat162 v2 = *(__nv_bfloat162*)p;
    const size_t slot_off = (size_t)a.cache_loc[tok] * a.kv_row_bytes;
    if (head >= a.qh + a.kvh) {  // v head: append only
        const int vh = head - a.qh - a.kvh;
        if (a.v_cache) *(__nv_bfloat162*)(a.v_cache + slot_off + vh * 128 + 4 * lane) = v2;
        return;
    }
    const float x0 = __bfloat162float(v2.x), x1 = __bfloat162float(v2.y);
    const float ms = warp_sum(x0 * x0 + x1 * x1) * (1.0f / 64.0f);
    const float scale = (head < a.qh ? a.q_scale : 1.0f) * (1.0f / sqrtf(ms + a.eps));
    float y0 = bf16_round(x0 * scale), y1 = bf16_round(x1 * scale);
    if (a.cos_sin) {
        const float c = a.cos_sin[tok * 64 + lane], s = a.cos_sin[tok * 64 + 32 + lane];
        const float r0 = fmaf(y0, c, -(y1 * s)), r1 = fmaf(y1, c, y0 * s);
        y0 = r0;
        y1 = r1;
    }
    const __nv_bfloat162 out = __floats2bfloat162_rn(y0, y1);
    *(__nv_bfloat162*)p = out;
    if (head >= a.qh && a.k_cache) *(__nv_bfloat162*)(a.k_cache + slot_off + (head - a.qh) * 128 + 4 * lane) = out;
}

// ---- launch helpers -----------------------------------------------------------------------------------------------------------

template <typename Kern, typename Args>
static cudaError_t launch1(Kern kern, dim3 grid, dim3 block, cudaStream_t stream, bool pdl, const Args& args) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, args);
}

cudaError_t resid_norm_launch(const NormArgs& a, cudaStream_t s, bool pdl) {
    return launch1(resid_norm_kernel, dim3(a.M), dim3(kNormThreads), s, pdl, a);
}
cudaError_t topk_launch(const TopkArgs& a, cudaStream_t s, bool pdl) {
    return launch1(topk_kernel, dim3(a.M), dim3(32), s, pdl, a);
}
cudaError_t nq_launch(const NqArgs& a, int M, cudaStream_t s, bool pdl) {
    return launch1(nq_kernel, dim3(M), dim3(256), s, pdl, a);
}
cudaError_t route_tables_launch(const int* ids, int E, int k, int b_live, RouteTables* rt, cudaStream_t s, bool pdl) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(128);
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, route_tables_kernel, ids, E, k, b_live, rt);
}
cudaError_t hrow_launch(const unsigned char* z_sf, const signed char* z_ex, int groups, int slots_live, int slots,
                        unsigned char* z_sfd, float* rowscale, cudaStream_t s, bool pdl) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(slots);
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, hrow_kernel, z_sf, z_ex, groups, slots_live, z_sfd, rowscale);
}
cudaError_t combine_launch(const CombineArgs& a, int M, cudaStream_t s, bool pdl) {
    return launch1(combine_kernel, dim3(M), dim3(256), s, pdl, a);
}
cudaError_t rowops_launch(const RowopsArgs& a, cudaStream_t s, bool pdl) {
    const int warps = a.M * (a.qh + 2 * a.kvh);
    return launch1(rowops_kernel, dim3((warps + 7) / 8), dim3(256), s, pdl, a);
}

}  // namespace mk
