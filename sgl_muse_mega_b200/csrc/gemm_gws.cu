// Skinny GEMM with its split-K partial sums in GLOBAL scratch (the stand-alone qkv head, mk_qkv_bind and
// mk_qkv_launch_static). Same weight streaming as gemm.cu; the K chunks of an N block meet through an f32 partial tile in
// caller-provided scratch and an arrival counter, and the last CTA to arrive sums the chunks in chunk order. It needs no
// thread-block cluster, so it takes any K split up to 16, at the price of one round trip through memory.
#include "stages.h"

namespace mk {

template <bool WF32>
struct GwsCfg {
    static constexpr int WN = WF32 ? 1 : 2;
    static constexpr int WK = WF32 ? 8 : 4;
    static constexpr int BN = 16 * WN;
    static constexpr int ES = WF32 ? 4 : 2;           // element bytes
    static constexpr int KSTEP = 64 / ES;             // k per step: 4 lanes x 16 bytes
    static constexpr int PAD = 64;                    // row padding (bytes) that spreads the B reads over the banks
};

__device__ __forceinline__ void gws_store(const GemmGwsArgs& a, int m, int n, float v) {
    const size_t off = (size_t)m * a.ldo + a.col0 + n;
    if (a.out_f32) {
        for (int i = 0; i < a.n_out; ++i) ((float*)a.out[i])[off] = v;
    } else {
        const bf16 b = __float2bfloat16_rn(v);
        for (int i = 0; i < a.n_out; ++i) ((bf16*)a.out[i])[off] = b;
    }
}

template <bool WF32>
__global__ void __launch_bounds__(256) skinny_gemm_gws_kernel(const GemmGwsArgs a) {
    using C = GwsCfg<WF32>;
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int s_last;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int wn = warp % C::WN, wk = warp / C::WN;
    const int nb = blockIdx.x, ky = blockIdx.y, ksplit = gridDim.y;
    const int KC = a.K / ksplit;
    const int k0 = ky * KC;
    const int row_bytes = KC * C::ES + C::PAD;
    float* red = reinterpret_cast<float*>(smem + 16 * row_bytes);  // [WK][WN][8][32]

    // weight loads do not depend on the predecessor: issue the first ones before the dependency wait
    const int kw = KC / C::WK;           // k per warp
    const int nsteps = kw / C::KSTEP;
    const int n0 = nb * C::BN + wn * 16;
    const unsigned char* wbase = (const unsigned char*)a.w;
    const unsigned char* w0 = wbase + ((size_t)(n0 + g) * a.ldw + k0 + wk * kw) * C::ES + t * 16;
    const unsigned char* w1 = w0 + (size_t)8 * a.ldw * C::ES;
    constexpr int U = 4;
    uint4 ra[U], rb[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
        if (u < nsteps) {
            ra[u] = ldg_stream16(w0 + u * 64);
            rb[u] = ldg_stream16(w1 + u * 64);
        }

    griddep_wait();
    // stage the activations: rows >= M are zero
    {
        const int chunks = KC * C::ES / 16;
        for (int i = tid; i < 16 * chunks; i += 256) {
            const int r = i / chunks, c = i - r * chunks;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < a.M) v = *(const uint4*)((const unsigned char*)a.x + ((size_t)r * a.ldx + k0) * C::ES + c * 16);
            *(uint4*)(smem + r * row_bytes + c * 16) = v;
        }
    }
    __syncthreads();

    float acc0[4] = {0, 0, 0, 0}, acc1[4] = {0, 0, 0, 0};
    const bool two = a.M > 8;
    const unsigned char* xs0 = smem + g * row_bytes + (wk * kw) * C::ES + t * 16;
    const unsigned char* xs1 = xs0 + 8 * row_bytes;
    for (int s = 0; s < nsteps; s += U) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (s + u < nsteps) {
                uint4 wa = ra[u], wb = rb[u];
                if (s + u + U < nsteps) {
                    ra[u] = ldg_stream16(w0 + (s + u + U) * 64);
                    rb[u] = ldg_stream16(w1 + (s + u + U) * 64);
                }
                const uint4 x0 = *(const uint4*)(xs0 + (s + u) * 64);
                if (WF32) {
                    wa.x &= 0xFFFFE000u; wa.y &= 0xFFFFE000u; wa.z &= 0xFFFFE000u; wa.w &= 0xFFFFE000u;
                    wb.x &= 0xFFFFE000u; wb.y &= 0xFFFFE000u; wb.z &= 0xFFFFE000u; wb.w &= 0xFFFFE000u;
                    mma_tf32_1688(acc0, wa.x, wb.x, wa.y, wb.y, x0.x, x0.y);
                    mma_tf32_1688(acc0, wa.z, wb.z, wa.w, wb.w, x0.z, x0.w);
                } else {
                    mma_bf16_16816(acc0, wa.x, wb.x, wa.y, wb.y, x0.x, x0.y);
                    mma_bf16_16816(acc0, wa.z, wb.z, wa.w, wb.w, x0.z, x0.w);
                }
                if (two) {
                    const uint4 x1 = *(const uint4*)(xs1 + (s + u) * 64);
                    if (WF32) {
                        mma_tf32_1688(acc1, wa.x, wb.x, wa.y, wb.y, x1.x, x1.y);
                        mma_tf32_1688(acc1, wa.z, wb.z, wa.w, wb.w, x1.z, x1.w);
                    } else {
                        mma_bf16_16816(acc1, wa.x, wb.x, wa.y, wb.y, x1.x, x1.y);
                        mma_bf16_16816(acc1, wa.z, wb.z, wa.w, wb.w, x1.z, x1.w);
                    }
                }
            }
        }
    }
    // meet the K warps in shared memory
    {
        float* r = red + ((wk * C::WN + wn) * 8) * 32 + lane;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            r[i * 32] = acc0[i];
            r[(4 + i) * 32] = acc1[i];
        }
    }
    __syncthreads();
    // element e of a row group: i = e / 32 (accumulator register), lane' = e % 32
    for (int e = tid; e < C::WN * 256; e += 256) {
        const int rn = e >> 8, i = (e >> 5) & 7, ln = e & 31;
        float v = 0.f;
#pragma unroll
        for (int k = 0; k < C::WK; ++k) v += red[((k * C::WN + rn) * 8 + i) * 32 + ln];
        const int gg = ln >> 2, tt = ln & 3;
        const int n = nb * C::BN + rn * 16 + gg + 8 * ((i >> 1) & 1);
        const int m = (i >> 2) * 8 + 2 * tt + (i & 1);
        if (ksplit == 1) {
            if (m < a.M) gws_store(a, m, n, v);
        } else {
            a.partial[((size_t)ky * 16 + m) * a.N + n] = v;
        }
    }
    if (ksplit == 1) return;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned old = atomicAdd(a.counter + nb, 1u);
        s_last = (old == (unsigned)(ksplit - 1));
        if (s_last) a.counter[nb] = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int e = tid; e < C::BN * 16; e += 256) {
        const int m = e / C::BN, n = nb * C::BN + (e % C::BN);
        if (m >= a.M) continue;
        float v = 0.f;
        for (int k = 0; k < ksplit; ++k) v += __ldcg(a.partial + ((size_t)k * 16 + m) * a.N + n);
        gws_store(a, m, n, v);
    }
}

// Picks the K split: chunks of at most `kc_max` elements that divide K and give every warp whole steps.
static int gws_pick_ksplit(int K, int kc_max, int wk, int kstep) {
    for (int ks = 1; ks <= 64; ++ks) {
        if (K % ks) continue;
        const int kc = K / ks;
        if (kc <= kc_max && kc % (wk * kstep) == 0) return ks;
    }
    return -1;
}

int gemm_gws_ksplit(bool wf32, int K) {
    return wf32 ? gws_pick_ksplit(K, 512, GwsCfg<true>::WK, GwsCfg<true>::KSTEP)
                : gws_pick_ksplit(K, 1024, GwsCfg<false>::WK, GwsCfg<false>::KSTEP);
}
int gemm_gws_bn(bool wf32) { return wf32 ? GwsCfg<true>::BN : GwsCfg<false>::BN; }

size_t gemm_gws_smem(bool wf32, int K, int ksplit) {
    const int es = wf32 ? 4 : 2, kc = K / ksplit;
    const int wn = wf32 ? 1 : 2, wk = wf32 ? 8 : 4;
    return (size_t)16 * (kc * es + 64) + (size_t)wk * wn * 8 * 32 * 4;
}

cudaError_t gemm_gws_prepare() {
    cudaError_t e = cudaFuncSetAttribute(skinny_gemm_gws_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(skinny_gemm_gws_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
}

cudaError_t gemm_gws_launch(const GemmGwsArgs& a, bool wf32, int ksplit, cudaStream_t stream, bool pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.N / gemm_gws_bn(wf32), ksplit, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.dynamicSmemBytes = gemm_gws_smem(wf32, a.K, ksplit);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return wf32 ? cudaLaunchKernelEx(&cfg, skinny_gemm_gws_kernel<true>, a)
                : cudaLaunchKernelEx(&cfg, skinny_gemm_gws_kernel<false>, a);
}

}  // namespace mk
