// Skinny GEMM for the verify window: out[m, n] = sum_k x[m, k] W[n, k] with M <= 16 rows of activations and a weight
// matrix that is read exactly once. Weight streaming bounds it and the weights never depend on the predecessor kernel,
// so the kernel is built around one idea: a CTA's WHOLE weight tile (BN rows x one K slice, at most 131 KB) is fetched
// into shared memory by bulk copies (one per weight row, the TMA engine without a tensor map) issued BEFORE the
// programmatic-dependent-launch wait. With one CTA per SM and a grid of at most one wave, the entire weight matrix is in
// flight or already on chip while the predecessor kernel is still running; after the wait only the activation slice, the
// MMAs from shared memory and the epilogue remain.
//
// MMA: mma.sync m16n8k16 (bf16) / m16n8k8 (tf32, low 13 mantissa bits of the f32 weights masked) with the weights as the
// 16-row operand and the window rows as the 8-column operand ("swap-AB"). K permutation: a thread's 16-byte shared-memory
// read covers 8 consecutive k of one weight row; the two MMAs it feeds take (k0 k1 | k2 k3) and (k4 k5 | k6 k7) as their
// (k, k+8) register pairs, and the B fragments are read with the same permutation, so the dot products are unchanged.
// Rows are padded by 64 bytes so that the 16-byte reads of a quarter warp fall into distinct banks.
//
// Work split: grid (N / BN, ksplit), one thread-block CLUSTER per N block along y. The 8 / WN warps per 16-row group
// split the K slice and meet in shared memory; the K slices of a cluster meet through distributed shared memory: CTA r
// sums, in slice order (a fixed order: results do not depend on timing), the window rows r, r + ksplit, ... of every
// CTA's partial tile and runs the epilogue for them. No partial sum touches global memory and there is no atomic.
//
// Epilogue mode 1 (the qkv head, BN = 64 = one head): bf16(acc), per-head qk norm (q scaled), interleaved-pair RoPE,
// K and V rows appended to the successor's pool                                  (test/reference/muse_spark.py:601-635).
#include "stages.h"
#include "umma.cuh"

namespace mk {

template <bool WF32>
struct GemmCfg {
    static constexpr int WN = WF32 ? 1 : 4;  // 16-row groups per CTA
    static constexpr int WK = 8 / WN;
    static constexpr int BN = 16 * WN;
    static constexpr int ES = WF32 ? 4 : 2;  // element bytes
    static constexpr int KSTEP = 64 / ES;    // k per step: 4 lanes x 16 bytes
    static constexpr int PAD = 64;           // row padding (bytes) that spreads the 16-byte reads over the banks
};

__device__ __forceinline__ void gemm_store(const GemmArgs& a, int m, int n, float v) {
    const size_t off = (size_t)m * a.ldo + a.col0 + n;
    if (a.out_f32) {
        for (int i = 0; i < a.n_out; ++i) ((float*)a.out[i])[off] = v;
    } else {
        const bf16 b = __float2bfloat16_rn(v);
        for (int i = 0; i < a.n_out; ++i) ((bf16*)a.out[i])[off] = b;
    }
}

__device__ __forceinline__ uint32_t cluster_map(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <bool WF32>
__global__ void __launch_bounds__(256) skinny_gemm_kernel(const GemmArgs a) {
    using C = GemmCfg<WF32>;
    constexpr int WN = C::WN;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint64_t bar;
    __shared__ int s_abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int wn = warp % WN, wk = warp / WN;
    const int nb = blockIdx.x, ky = blockIdx.y, ksplit = a.ksplit;
    const int KC = a.K / ksplit;
    const int k0 = ky * KC;
    const int row_bytes = KC * C::ES + C::PAD;
    unsigned char* wsm = smem;                                      // [BN][row_bytes] the weight tile
    unsigned char* xsm = smem + C::BN * row_bytes;                  // [16][row_bytes] the activation slice
    float* red = reinterpret_cast<float*>(xsm + 16 * row_bytes);    // [WK][WN][8][32]
    float* tile = red + 8 * 8 * 32;                                 // [BN][16] this CTA's partial sums

    // the whole weight tile, one bulk copy per row, before the wait on the predecessor
    if (tid == 0) {
        s_abort = 0;
        umma::mbar_init(&bar, 1);
        umma::mbar_fence_init();
        // the last tile of an N that is not a multiple of BN has fewer rows: rows past N are neither fetched nor stored
        const int valid = min(C::BN, a.N - nb * C::BN);
        umma::mbar_arrive_expect_tx(&bar, (uint32_t)(valid * KC * C::ES));
    }
    __syncthreads();
    if (tid < C::BN && nb * C::BN + tid < a.N)
        umma::bulk_g2s(wsm + tid * row_bytes, (const unsigned char*)a.w + ((size_t)(nb * C::BN + tid) * a.ldw + k0) * C::ES,
                       (uint32_t)(KC * C::ES), &bar);

    griddep_wait();
    // stage the activations with asynchronous 16-byte copies: rows >= M are zero-filled
    {
        const int chunks = KC * C::ES / 16;
        for (int i = tid; i < 16 * chunks; i += 256) {
            const int r = i / chunks, c = i - r * chunks;
            const bool ok = r < a.M;
            cp_async16(xsm + r * row_bytes + c * 16, (const unsigned char*)a.x + ((size_t)(ok ? r : 0) * a.ldx + k0) * C::ES + c * 16, ok);
        }
        cp_async_commit();
        cp_async_wait<0>();
    }
    if (!umma::mbar_wait(&bar, 0, &s_abort)) {
        // the copies never landed: record it and go on (the outputs of this tile are then meaningless, the status says so)
        if (atomicExch(&s_abort, 1) == 0 && a.status != nullptr) {
            a.status[1] = 200;
            a.status[2] = (int)blockIdx.x;
            a.status[3] = (int)blockIdx.y;
            __threadfence();
            a.status[0] = 3;
        }
    }
    __syncthreads();

    const int kw = KC / C::WK;  // k per warp
    const int nsteps = kw / C::KSTEP;
    float acc0[4] = {0, 0, 0, 0}, acc1[4] = {0, 0, 0, 0};
    const bool two = a.M > 8;
    const unsigned char* wa0 = wsm + (wn * 16 + g) * row_bytes + (wk * kw) * C::ES + t * 16;
    const unsigned char* wa1 = wa0 + 8 * row_bytes;
    const unsigned char* xs0 = xsm + g * row_bytes + (wk * kw) * C::ES + t * 16;
    const unsigned char* xs1 = xs0 + 8 * row_bytes;
#pragma unroll 4
    for (int s = 0; s < nsteps; ++s) {
        uint4 wa = *(const uint4*)(wa0 + s * 64), wb = *(const uint4*)(wa1 + s * 64);
        const uint4 x0 = *(const uint4*)(xs0 + s * 64);
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
            const uint4 x1 = *(const uint4*)(xs1 + s * 64);
            if (WF32) {
                mma_tf32_1688(acc1, wa.x, wb.x, wa.y, wb.y, x1.x, x1.y);
                mma_tf32_1688(acc1, wa.z, wb.z, wa.w, wb.w, x1.z, x1.w);
            } else {
                mma_bf16_16816(acc1, wa.x, wb.x, wa.y, wb.y, x1.x, x1.y);
                mma_bf16_16816(acc1, wa.z, wb.z, wa.w, wb.w, x1.z, x1.w);
            }
        }
    }
    // meet the K warps of the CTA in shared memory
    {
        float* r = red + ((wk * WN + wn) * 8) * 32 + lane;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            r[i * 32] = acc0[i];
            r[(4 + i) * 32] = acc1[i];
        }
    }
    __syncthreads();
    // accumulator register i of lane ln of row group rn holds (row ln/4 + 8 (i/2 % 2), window row 8 (i/4) + 2 (ln%4) + i%2)
    for (int e = tid; e < WN * 256; e += 256) {
        const int rn = e >> 8, i = (e >> 5) & 7, ln = e & 31;
        float v = 0.f;
#pragma unroll
        for (int k = 0; k < C::WK; ++k) v += red[((k * WN + rn) * 8 + i) * 32 + ln];
        const int n = rn * 16 + (ln >> 2) + 8 * ((i >> 1) & 1);
        const int m = (i >> 2) * 8 + 2 * (ln & 3) + (i & 1);
        tile[n * 16 + m] = v;
    }
    if (ksplit > 1) cluster_sync_all();
    else __syncthreads();

    // the K slices of the cluster meet: this CTA finishes the window rows ky, ky + ksplit, ...; one warp per row
    const uint32_t tile_addr = (uint32_t)__cvta_generic_to_shared(tile);
    for (int m = ky + ksplit * warp; m < a.M; m += ksplit * 8) {
        auto total = [&](int n) {
            if (ksplit == 1) return tile[n * 16 + m];
            float v = 0.f;
            for (int c = 0; c < ksplit; ++c) v += ld_cluster_f32(cluster_map(tile_addr + (n * 16 + m) * 4, c));
            return v;
        };
        if (a.mode == 0) {
            for (int n = lane; n < C::BN; n += 32)
                if (nb * C::BN + n < a.N) {
                    const float v = total(n);
                    gemm_store(a, m, nb * C::BN + n, v);
                    if (a.score != nullptr) {
                        // the router's selection score, here because this epilogue has a thread per logit while the
                        // routing kernel has one warp per row: sigmoid in f64 rounded to f32, plus the expert's bias
                        const int e = nb * C::BN + n;
                        const float s = (float)(1.0 / (1.0 + exp(-((double)v * a.score_mult))));
                        a.score[(size_t)m * a.N + e] = s + a.score_bias[e];
                    }
                }
        } else {
            // one head: lane owns the pair (2 lane, 2 lane + 1)
            const int head = nb;
            float y0 = bf16_round(total(2 * lane)), y1 = bf16_round(total(2 * lane + 1));
            bf16* orow = (bf16*)a.out[0] + (size_t)m * a.ldo + head * kHeadDim + 2 * lane;
            const size_t slot_off = (size_t)a.cache_loc[m] * a.kv_row_bytes;
            if (head < a.qh + a.kvh) {
                const float ms = warp_sum(y0 * y0 + y1 * y1) * (1.0f / 64.0f);
                const float scale = (head < a.qh ? a.q_scale : 1.0f) * (1.0f / sqrtf(ms + a.eps));
                y0 = bf16_round(y0 * scale);
                y1 = bf16_round(y1 * scale);
                if (a.cos_sin) {
                    const float c = a.cos_sin[m * 64 + lane], s = a.cos_sin[m * 64 + 32 + lane];
                    const float r0 = fmaf(y0, c, -(y1 * s)), r1 = fmaf(y1, c, y0 * s);
                    y0 = r0;
                    y1 = r1;
                }
            }
            const __nv_bfloat162 o2 = __floats2bfloat162_rn(y0, y1);
            *(__nv_bfloat162*)orow = o2;
            if (head >= a.qh && head < a.qh + a.kvh && a.k_cache)
                *(__nv_bfloat162*)(a.k_cache + slot_off + (head - a.qh) * 128 + 4 * lane) = o2;
            if (head >= a.qh + a.kvh && head < a.qh + 2 * a.kvh && a.v_cache)
                *(__nv_bfloat162*)(a.v_cache + slot_off + (head - a.qh - a.kvh) * 128 + 4 * lane) = o2;
        }
    }
    // no CTA leaves while another may still read its partial tile
    if (ksplit > 1) cluster_sync_all();
    xchg_signal(a.sig);
}

// ---- host side ----

static size_t smem_bytes(bool wf32, int K, int ksplit) {
    const int es = wf32 ? 4 : 2, kc = K / ksplit, bn = wf32 ? 16 : 64;
    return (size_t)(bn + 16) * (kc * es + 64) + (size_t)8 * 8 * 32 * 4 + (size_t)bn * 16 * 4;
}

// Chooses the K split of one GEMM (the tile height is fixed by the weight type: 64 rows bf16, 16 rows f32): among the
// splits whose weight tile and activation slice fit shared memory and give every warp whole 64-byte steps, the largest
// that keeps the grid within one wave of `max_ctas` CTAs, else the smallest (fewest CTAs beyond one wave).
int gemm_plan(bool wf32, int mode, int N, int K, int max_ctas, int* wn_out, int* ksplit_out) {
    const int wn = wf32 ? 1 : 4;
    const int bn = 16 * wn, wk = 8 / wn, kstep = wf32 ? 16 : 32;
    if (mode == 1 && N % bn) return -1;  // a head tile must be whole; plain tiles may have a short last tile
    const int nblocks = (N + bn - 1) / bn;
    int best = -1, smallest = -1;
    for (int ks = 8; ks >= 1; ks >>= 1) {
        if (K % ks) continue;
        const int kc = K / ks;
        if (kc % (wk * kstep)) continue;
        if (smem_bytes(wf32, K, ks) > 220 * 1024) continue;
        smallest = ks;
        if (best < 0 && (long long)nblocks * ks <= max_ctas) best = ks;
    }
    const int ks = best > 0 ? best : smallest;
    if (ks < 0) return -1;
    *wn_out = wn;
    *ksplit_out = ks;
    return 0;
}

size_t gemm_smem(const GemmArgs& a, bool wf32) { return smem_bytes(wf32, a.K, a.ksplit); }
int gemm_grid(const GemmArgs& a) { return ((a.N + 16 * a.wn - 1) / (16 * a.wn)) * a.ksplit; }

cudaError_t gemm_prepare() {
    cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(skinny_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
}

cudaError_t gemm_launch(const GemmArgs& a, bool wf32, cudaStream_t stream, bool pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((a.N + 16 * a.wn - 1) / (16 * a.wn), a.ksplit, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.dynamicSmemBytes = gemm_smem(a, wf32);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (a.ksplit > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = a.ksplit;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return wf32 ? cudaLaunchKernelEx(&cfg, skinny_gemm_kernel<true>, a) : cudaLaunchKernelEx(&cfg, skinny_gemm_kernel<false>, a);
}

}  // namespace mk
