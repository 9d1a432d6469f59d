// The MoE phase on CUDA cores (general shapes): g1 = gate/up rows of the rank's intermediate slice with the SwiGLU and
// the per-16 requantisation of h in the epilogue, g2 = the rank's output rows over the full gathered h row.
//
// One CTA per (active expert, group of 16 features / 16 output rows). The routed rows of the expert (at most 16, a row
// picks an expert once) are dequantised into shared memory as f16 (a code times its block scale is exact in f16), each
// warp walks whole weight rows with 16-byte loads and keeps one f32 accumulator per routed row.
// Arithmetic contract: test/reference/muse_spark.py:438-563 (NVFP4) and :566-584 (bf16 experts);
// reference kernels: sm103/kernels/moe.cuh:1018-2458.
#include "stages.h"

namespace mk {


// dot products of one NVFP4 weight row against n_tok f16 rows of shared memory; K elements; lane-strided 32-element chunks
template <int MAXT>
__device__ __forceinline__ void fp4_row_dot(const unsigned char* wq, const unsigned char* wsf, int K, const __half* xs, int ldx,
                                            int n_tok, float (&acc)[MAXT]) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int i = 0; i < MAXT; ++i) acc[i] = 0.f;
    for (int k0 = lane * 32; k0 < K; k0 += 1024) {
        const uint4 c = ldg_stream16(wq + k0 / 2);
        const uint32_t sfw = *(const unsigned short*)(wsf + k0 / 16);
        const float s0 = e4m3_to_float(sfw & 0xFF), s1 = e4m3_to_float(sfw >> 8);
        float w[32];
        const uint32_t cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
        for (int i = 0; i < 32; ++i) w[i] = e2m1_to_float((cw[i >> 3] >> (4 * (i & 7))) & 15u);
        for (int tk = 0; tk < n_tok; ++tk) {
            const __half2* xp = (const __half2*)(xs + (size_t)tk * ldx + k0);
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 x = __half22float2(xp[i]);
                a0 = fmaf(w[2 * i], x.x, a0);
                a0 = fmaf(w[2 * i + 1], x.y, a0);
            }
#pragma unroll
            for (int i = 8; i < 16; ++i) {
                const float2 x = __half22float2(xp[i]);
                a1 = fmaf(w[2 * i], x.x, a1);
                a1 = fmaf(w[2 * i + 1], x.y, a1);
            }
#pragma unroll
            for (int i = 0; i < MAXT; ++i)
                if (i == tk) acc[i] += a0 * s0 + a1 * s1;
        }
    }
#pragma unroll
    for (int i = 0; i < MAXT; ++i) acc[i] = warp_sum(acc[i]);
}

template <int MAXT>
__device__ __forceinline__ void bf16_row_dot(const bf16* w, int K, const bf16* xs, int ldx, int n_tok, float (&acc)[MAXT]) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int i = 0; i < MAXT; ++i) acc[i] = 0.f;
    for (int k0 = lane * 8; k0 < K; k0 += 256) {
        const uint4 c = ldg_stream16(w + k0);
        const __nv_bfloat162* wp = (const __nv_bfloat162*)&c;
        float wf[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(wp[i]);
            wf[2 * i] = f.x;
            wf[2 * i + 1] = f.y;
        }
        for (int tk = 0; tk < n_tok; ++tk) {
            const __nv_bfloat162* xp = (const __nv_bfloat162*)(xs + (size_t)tk * ldx + k0);
            float a0 = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 x = __bfloat1622float2(xp[i]);
                a0 = fmaf(wf[2 * i], x.x, a0);
                a0 = fmaf(wf[2 * i + 1], x.y, a0);
            }
#pragma unroll
            for (int i = 0; i < MAXT; ++i)
                if (i == tk) acc[i] += a0;
        }
    }
#pragma unroll
    for (int i = 0; i < MAXT; ++i) acc[i] = warp_sum(acc[i]);
}

// amax 2^-e in (1024, 2048], one octave up when the mantissa exceeds 1.3125; floor -120   (muse_spark.py:438-444)
__device__ __forceinline__ int prov_exp(float amax) {
    const int b = __float_as_int(amax);
    const int bump = ((b & 0x7FFFFF) > 0x280000) || (b > 0x7F800000);
    return max((b >> 23) - 138 + bump, -120);
}

// g1: grid (I_s / 16, max_active), 256 threads, dynamic smem = 16 rows x P f16 (bf16 variant: bf16) + accumulators
__global__ void __launch_bounds__(256) g1_kernel(const ExpertArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    griddep_wait();
    const int ai = blockIdx.y;
    if (ai >= a.rt->n_active) {  // an idle CTA still arrives at the exchange
        xchg_signal(a.sig_g1);
        return;
    }
    const int e = a.rt->act_e[ai], s0 = a.rt->act_off[ai], n_tok = a.rt->act_off[ai + 1] - s0;
    const int fg = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float* accs = (float*)smem;                       // [32 rows][16 tokens]
    unsigned char* xs = smem + 32 * 16 * sizeof(float);  // [n_tok][P] 2-byte elements
    // stage the routed rows
    if (a.wbf16) {
        for (int i = tid; i < n_tok * (a.P / 8); i += 256) {
            const int tk = i / (a.P / 8), c = i % (a.P / 8);
            const int tok = a.rt->slot[s0 + tk] / a.topk;
            ((uint4*)xs)[(size_t)tk * (a.P / 8) + c] = ((const uint4*)a.xq)[(size_t)tok * (a.P / 8) + c];
        }
    } else {
        const int groups = a.P / 16;
        for (int i = tid; i < n_tok * groups; i += 256) {
            const int tk = i / groups, gi = i % groups;
            const int tok = a.rt->slot[s0 + tk] / a.topk;
            const uint2 c = *(const uint2*)(a.xq + (size_t)tok * (a.P / 2) + gi * 8);
            const float sf = e4m3_to_float(a.x_sf[(size_t)tok * groups + gi]);
            __half* o = (__half*)xs + (size_t)tk * a.P + gi * 16;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                o[j] = __float2half_rn(e2m1_to_float((c.x >> (4 * j)) & 15u) * sf);
                o[8 + j] = __float2half_rn(e2m1_to_float((c.y >> (4 * j)) & 15u) * sf);
            }
        }
    }
    __syncthreads();
    // 32 weight rows: 16 gate then 16 up features of this group; 4 rows per warp
    for (int ri = warp * 4; ri < warp * 4 + 4; ++ri) {
        const int up = ri >> 4, f = fg * 16 + (ri & 15);
        float acc[kMaxRows];
        if (a.wbf16) {
            const bf16* w = (const bf16*)(up ? a.w1_up : a.w1_gate) + ((size_t)e * a.I_s + f) * a.P;
            bf16_row_dot<kMaxRows>(w, a.P, (const bf16*)xs, a.P, n_tok, acc);
        } else {
            const unsigned char* wq = (up ? a.w1_up : a.w1_gate) + ((size_t)e * a.I_s + f) * (a.P / 2);
            const unsigned char* ws = (up ? a.w1_up_sf : a.w1_gate_sf) + ((size_t)e * a.I_s + f) * (a.P / 16);
            fp4_row_dot<kMaxRows>(wq, ws, a.P, (const __half*)xs, a.P, n_tok, acc);
        }
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < kMaxRows; ++i) accs[ri * 16 + i] = acc[i];
        }
    }
    __syncthreads();
    // epilogue: one thread per routed row handles the 16 features of the group
    if (tid < n_tok) {
        const int slot = a.rt->slot[s0 + tid], tok = slot / a.topk;
        float z[16];
        if (a.wbf16) {
            bf16 out[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float g = bf16_round(accs[i * 16 + tid]), u = bf16_round(accs[(16 + i) * 16 + tid]);
                out[i] = __float2bfloat16_rn((g / (1.0f + expf(-g))) * u);
            }
            for (int p = 0; p < a.n_peer; ++p) {
                bf16* dst = (bf16*)a.z_peer[p] + (size_t)slot * a.I + a.rank * a.I_s + fg * 16;
#pragma unroll
                for (int i = 0; i < 16; ++i) dst[i] = out[i];
            }
        } else {
        const float a1 = a.g1_alphas[e] * a.x_scale[tok], c1 = a.g1_scale_c[e];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float g = bf16_round(accs[i * 16 + tid] * a1), u = bf16_round(accs[(16 + i) * 16 + tid] * a1);
            z[i] = ((g / (1.0f + expf(-g))) * u) * c1;
            amax = fmaxf(amax, fabsf(z[i]));
        }
        const int eg = prov_exp(amax);
        const float down = __uint_as_float((uint32_t)(127 - eg) << 23);
        const uint32_t sfb = float_to_e4m3((amax * down) * (1.0f / 6.0f));
        const float d = e4m3_to_float(sfb);
        const float inv = d > 0.f ? 1.0f / d : 0.f;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            lo |= float_to_e2m1((z[i] * down) * inv) << (4 * i);
            hi |= float_to_e2m1((z[8 + i] * down) * inv) << (4 * i);
        }
        const int gcol = (a.rank * a.I_s) / 16 + fg;
        for (int p = 0; p < a.n_peer; ++p) {
            *(uint2*)(a.z_peer[p] + (size_t)slot * (a.I / 2) + gcol * 8) = make_uint2(lo, hi);
            a.zsf_peer[p][(size_t)slot * (a.I / 16) + gcol] = (unsigned char)sfb;
            a.zex_peer[p][(size_t)slot * (a.I / 16) + gcol] = (signed char)eg;
        }
        }
    }
    xchg_signal(a.sig_g1);
}

// g2: grid (H_s / 16, max_active), 256 threads, dynamic smem = 16 rows x I two-byte elements + accumulators
__global__ void __launch_bounds__(256) g2_kernel(const ExpertArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    griddep_wait();
    xchg_wait(a.wait_g2);
    const int ai = blockIdx.y;
    if (ai >= a.rt->n_active) {
        xchg_signal(a.sig_g2);
        return;
    }
    const int e = a.rt->act_e[ai], s0 = a.rt->act_off[ai], n_tok = a.rt->act_off[ai + 1] - s0;
    const int rg = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float* accs = (float*)smem;  // [16 rows][16 tokens]
    unsigned char* xs = smem + 16 * 16 * sizeof(float);
    if (a.wbf16) {
        for (int i = tid; i < n_tok * (a.I / 8); i += 256) {
            const int tk = i / (a.I / 8), c = i % (a.I / 8);
            const int slot = a.rt->slot[s0 + tk];
            ((uint4*)xs)[(size_t)tk * (a.I / 8) + c] = ((const uint4*)a.z)[(size_t)slot * (a.I / 8) + c];
        }
    } else {
        const int groups = a.I / 16;
        for (int i = tid; i < n_tok * groups; i += 256) {
            const int tk = i / groups, gi = i % groups;
            const int slot = a.rt->slot[s0 + tk];
            const uint2 c = *(const uint2*)(a.z + (size_t)slot * (a.I / 2) + gi * 8);
            const float sf = e4m3_to_float(a.z_sfd[(size_t)slot * groups + gi]);
            __half* o = (__half*)xs + (size_t)tk * a.I + gi * 16;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                o[j] = __float2half_rn(e2m1_to_float((c.x >> (4 * j)) & 15u) * sf);
                o[8 + j] = __float2half_rn(e2m1_to_float((c.y >> (4 * j)) & 15u) * sf);
            }
        }
    }
    __syncthreads();
    for (int ri = warp * 2; ri < warp * 2 + 2; ++ri) {
        const int n = rg * 16 + ri;
        float acc[kMaxRows];
        if (a.wbf16) {
            bf16_row_dot<kMaxRows>((const bf16*)a.w2 + ((size_t)e * a.H_s + n) * a.I, a.I, (const bf16*)xs, a.I, n_tok, acc);
        } else {
            fp4_row_dot<kMaxRows>(a.w2 + ((size_t)e * a.H_s + n) * (a.I / 2), a.w2_sf + ((size_t)e * a.H_s + n) * (a.I / 16),
                                  a.I, (const __half*)xs, a.I, n_tok, acc);
        }
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < kMaxRows; ++i) accs[ri * 16 + i] = acc[i];
        }
    }
    __syncthreads();
    if (tid < n_tok * 16) {
        const int tk = tid / 16, ri = tid % 16;
        const int slot = a.rt->slot[s0 + tk];
        float v = accs[ri * 16 + tk];
        if (!a.wbf16) v = (v * a.rowscale[slot]) * a.g2_alphas[e];
        const bf16 b = __float2bfloat16_rn(v);
        for (int p = 0; p < a.n_peer; ++p) a.zb_peer[p][(size_t)slot * a.P + a.rank * a.H_s + rg * 16 + ri] = b;
    }
    xchg_signal(a.sig_g2);
}

// ---- bf16 experts (the model's first and last layer) --------------------------------------------------------------------------
// Weight streaming at M <= 16 rows per expert (1.3 rows on average): what matters is bytes in flight. These kernels keep
// nothing in shared memory but the routed rows' addresses, so eight 256-thread CTAs fit an SM, and a lane requests four
// 16-byte pieces of its weight row before it uses the first; the routed activation rows (<= 16 x 8 KB, shared by every CTA
// of the expert) come through L1. One warp per weight row (g2) or per feature's gate and up rows (g1).
template <int MAXT>
__device__ __forceinline__ void bf16_row_dot_global(const bf16* __restrict__ w, int K, const bf16* const* xrow, int n_tok,
                                                    float (&acc)[MAXT]) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int i = 0; i < MAXT; ++i) acc[i] = 0.f;
    for (int k0 = lane * 8; k0 < K; k0 += 1024) {
        uint4 c[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (k0 + u * 256 < K) c[u] = ldg_stream16(w + k0 + u * 256);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (k0 + u * 256 >= K) break;
            const __nv_bfloat162* wp = (const __nv_bfloat162*)&c[u];
            float wf[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(wp[i]);
                wf[2 * i] = f.x;
                wf[2 * i + 1] = f.y;
            }
            for (int tk = 0; tk < n_tok; ++tk) {
                const uint4 xv = __ldg((const uint4*)(xrow[tk] + k0 + u * 256));
                const __nv_bfloat162* xp = (const __nv_bfloat162*)&xv;
                float a0 = 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 x = __bfloat1622float2(xp[i]);
                    a0 = fmaf(wf[2 * i], x.x, a0);
                    a0 = fmaf(wf[2 * i + 1], x.y, a0);
                }
#pragma unroll
                for (int i = 0; i < MAXT; ++i)
                    if (i == tk) acc[i] += a0;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < MAXT; ++i) acc[i] = warp_sum(acc[i]);
}

constexpr int kBf16Feat = 16;  // features (g1) or output rows (g2) per CTA: two per warp

// g1, bf16: grid (I_s / 16, max_active). z[slot, rank I_s + f] = bf16(silu(bf16(gate . x)) bf16(up . x)) to every peer.
__global__ void __launch_bounds__(256) g1_bf16_kernel(const ExpertArgs a) {
    __shared__ const bf16* xrow[kMaxRows];
    __shared__ int slots[kMaxRows];
    griddep_wait();
    const int ai = blockIdx.y;
    if (ai >= a.rt->n_active) {
        xchg_signal(a.sig_g1);
        return;
    }
    const int e = a.rt->act_e[ai], s0 = a.rt->act_off[ai], n_tok = a.rt->act_off[ai + 1] - s0;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < n_tok) {
        slots[tid] = a.rt->slot[s0 + tid];
        xrow[tid] = (const bf16*)a.xq + (size_t)(slots[tid] / a.topk) * a.P;
    }
    __syncthreads();
    for (int j = 0; j < kBf16Feat / 8; ++j) {
        const int f = blockIdx.x * kBf16Feat + warp * (kBf16Feat / 8) + j;
        float g[kMaxRows], u[kMaxRows];
        bf16_row_dot_global<kMaxRows>((const bf16*)a.w1_gate + ((size_t)e * a.I_s + f) * a.P, a.P, xrow, n_tok, g);
        bf16_row_dot_global<kMaxRows>((const bf16*)a.w1_up + ((size_t)e * a.I_s + f) * a.P, a.P, xrow, n_tok, u);
        float gv = 0.f, uv = 0.f;
#pragma unroll
        for (int i = 0; i < kMaxRows; ++i)
            if (i == lane) { gv = g[i]; uv = u[i]; }
        if (lane < n_tok) {
            gv = bf16_round(gv);
            uv = bf16_round(uv);
            const bf16 out = __float2bfloat16_rn((gv / (1.0f + expf(-gv))) * uv);
            const size_t off = (size_t)slots[lane] * a.I + a.rank * a.I_s + f;
            for (int p = 0; p < a.n_peer; ++p) ((bf16*)a.z_peer[p])[off] = out;
        }
    }
    xchg_signal(a.sig_g1);
}

// g2, bf16: grid (H_s / 16, max_active). zb[slot, rank H_s + n] = bf16(w2[n] . z[slot]) to every peer.
__global__ void __launch_bounds__(256) g2_bf16_kernel(const ExpertArgs a) {
    __shared__ const bf16* xrow[kMaxRows];
    __shared__ int slots[kMaxRows];
    griddep_wait();
    xchg_wait(a.wait_g2);
    const int ai = blockIdx.y;
    if (ai >= a.rt->n_active) {
        xchg_signal(a.sig_g2);
        return;
    }
    const int e = a.rt->act_e[ai], s0 = a.rt->act_off[ai], n_tok = a.rt->act_off[ai + 1] - s0;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < n_tok) {
        slots[tid] = a.rt->slot[s0 + tid];
        xrow[tid] = (const bf16*)a.z + (size_t)slots[tid] * a.I;
    }
    __syncthreads();
    for (int j = 0; j < kBf16Feat / 8; ++j) {
        const int n = blockIdx.x * kBf16Feat + warp * (kBf16Feat / 8) + j;
        float acc[kMaxRows];
        bf16_row_dot_global<kMaxRows>((const bf16*)a.w2 + ((size_t)e * a.H_s + n) * a.I, a.I, xrow, n_tok, acc);
        float v = 0.f;
#pragma unroll
        for (int i = 0; i < kMaxRows; ++i)
            if (i == lane) v = acc[i];
        if (lane < n_tok) {
            const bf16 b = __float2bfloat16_rn(v);
            const size_t off = (size_t)slots[lane] * a.P + a.rank * a.H_s + n;
            for (int p = 0; p < a.n_peer; ++p) a.zb_peer[p][off] = b;
        }
    }
    xchg_signal(a.sig_g2);
}

size_t g1_smem(int P) { return 32 * 16 * sizeof(float) + (size_t)kMaxRows * P * 2; }
size_t g2_smem(int I) { return 16 * 16 * sizeof(float) + (size_t)kMaxRows * I * 2; }

cudaError_t experts_prepare() {
    cudaError_t e = cudaFuncSetAttribute(g1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(g2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
}

static cudaError_t launch_e(void (*kern)(const ExpertArgs), dim3 grid, size_t smem, cudaStream_t s, bool pdl, const ExpertArgs& a) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, a);
}

cudaError_t g1_launch(const ExpertArgs& a, int max_active, cudaStream_t s, bool pdl) {
    if (a.wbf16 && a.P % 8 == 0) return launch_e(g1_bf16_kernel, dim3(a.I_s / kBf16Feat, max_active), 0, s, pdl, a);
    return launch_e(g1_kernel, dim3(a.I_s / 16, max_active), g1_smem(a.P), s, pdl, a);
}
cudaError_t g2_launch(const ExpertArgs& a, int max_active, cudaStream_t s, bool pdl) {
    if (a.wbf16 && a.I % 8 == 0) return launch_e(g2_bf16_kernel, dim3(a.H_s / kBf16Feat, max_active), 0, s, pdl, a);
    return launch_e(g2_kernel, dim3(a.H_s / 16, max_active), g2_smem(a.I), s, pdl, a);
}

}  // namespace mk
