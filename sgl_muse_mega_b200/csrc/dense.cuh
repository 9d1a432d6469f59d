// The tensor-core dense engine: tile constants, the stream-K work split, the tcgen05 wrappers, the epilogues over a finished
// tile and the four roles (weight producer, MMA issuer, activation stager, epilogue) as device functions that carry their
// pipeline state from one GEMM stage of a kernel to the next. dense.cu builds the one-stage kernel from them, fused.cuh the
// kernels that chain two GEMM stages with the row work between them. See dense.cu for the design.
#pragma once

#include "draft_rows.cuh"
#include "umma.cuh"

// Trace builds (-DDENSE_TRACE): every CTA of a stand-alone dense launch stamps its milestones (global timer, 16 words a
// CTA) into a device array: 0 entry, 1 set up, 2 last weight stage issued, 3 programmatic wait returned (stager), 4 first
// rows staged, 5 first stage landed, 6 last MMA committed, 7 first accumulators complete, 8 epilogues done, 9 torn down,
// 10 first finish started.
#ifdef DENSE_TRACE
namespace mk {
static __device__ unsigned long long g_dense_trace[8][160][16];  // one copy per translation unit: dense.cu's is read
}
#define DT(slot)                                                                       \
    {                                                                                  \
        unsigned long long t_;                                                         \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                         \
        if (c.trace_id >= 0) mk::g_dense_trace[c.trace_id][blockIdx.x][(slot)] = t_;  \
    }
#else
#define DT(slot)
#endif

namespace mk {

using namespace umma;

constexpr int kDThreads = 256;
constexpr uint32_t kAtomW = 128 * 128;   // 128 weight rows x 128 bytes
constexpr uint32_t kStageW = 2 * kAtomW;
constexpr uint32_t kAtomX = 16 * 128;    // 16 window rows x 128 bytes
constexpr uint32_t kStageX = 2 * kAtomX;
constexpr int kTileLd = 132;             // floats per row of the epilogue tile (16 rows x 128 columns, padded)
constexpr uint32_t kDTmemCols = 32;      // two accumulators of 16 columns
constexpr int kXDepth = 3;               // activation stages a stager thread keeps in flight
constexpr int kDenseMaxGrid = 148;

struct Unit {
    int gi, tile, k0, k1, slot, n;
};

__device__ __forceinline__ int stages_of(const SegGemm& g) { return g.K * (g.f32 ? 4 : 2) / 256; }
__device__ __forceinline__ int tiles_of(const SegGemm& g) { return (g.N + 127) / 128; }

// One CTA's share of a GEMM stage: stage units [lo, hi) of the T units of the stage's one or two GEMMs (T0 of them the
// first GEMM's), cut evenly over the G CTAs. 32-bit arithmetic: the host refuses a stage with T x G >= 2^31.
struct Plan {
    uint32_t T0, T, G, lo, hi;
};
__device__ __forceinline__ Plan plan_of(const SegGemmArgs& a) {
    Plan p;
    p.T0 = (uint32_t)(tiles_of(a.g[0]) * stages_of(a.g[0]));
    p.T = p.T0 + (a.n_gemm > 1 ? (uint32_t)(tiles_of(a.g[1]) * stages_of(a.g[1])) : 0u);
    p.G = gridDim.x;
    p.lo = blockIdx.x * p.T / p.G;
    p.hi = (blockIdx.x + 1) * p.T / p.G;
    return p;
}
// the CTA whose range holds stage unit s: the largest c with floor(c T / G) <= s
__device__ __forceinline__ int cta_of(uint32_t s, uint32_t T, uint32_t G) { return (int)(((s + 1) * G + T - 1) / T - 1); }

__device__ __forceinline__ Unit unit_at(const SegGemmArgs& a, const Plan& pl, uint32_t p) {
    Unit u;
    u.gi = p >= pl.T0 ? 1 : 0;
    const uint32_t base = u.gi ? pl.T0 : 0u;
    const uint32_t KS = (uint32_t)stages_of(a.g[u.gi]);
    const uint32_t rel = p - base;
    u.tile = (int)(rel / KS);
    u.k0 = (int)(rel - (uint32_t)u.tile * KS);
    const uint32_t left = pl.hi - p;
    u.k1 = (int)(left < KS - (uint32_t)u.k0 ? (uint32_t)u.k0 + left : KS);
    const uint32_t first = base + (uint32_t)u.tile * KS;
    const int c0 = cta_of(first, pl.T, pl.G), c1 = cta_of(first + KS - 1, pl.T, pl.G);
    u.slot = (int)blockIdx.x - c0;
    u.n = c1 - c0 + 1;
    return u;
}

__device__ __forceinline__ void dense_abort(int* status, volatile int* abort, int where, int observed) {
    if (atomicExch((int*)abort, 1) == 0 && status != nullptr && atomicCAS(status, 0, 3) == 0) {
        status[1] = where;
        status[2] = (int)blockIdx.x;
        status[3] = observed;
        status[4] = 0;
    }
}

__host__ __device__ constexpr uint32_t idesc_dense(bool tf32) {
    // f32 accumulator (bit 4), A and B formats at [7,10) / [10,13) (1 = bf16, 2 = tf32), both K-major, N = 16, M = 128
    return (1u << 4) | ((tf32 ? 2u : 1u) << 7) | ((tf32 ? 2u : 1u) << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ void mma_bf16(uint32_t d, uint64_t ad, uint64_t bd, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(d), "l"(ad), "l"(bd), "r"(idesc_dense(false)), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void mma_tf32(uint32_t d, uint64_t ad, uint64_t bd, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(d), "l"(ad), "l"(bd), "r"(idesc_dense(true)), "r"(acc)
        : "memory");
}

__device__ __forceinline__ uint4 pack8f(const float* f) {
    uint4 v;
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return v;
}

// ---- epilogues over the finished tile (16 window rows x 128 weight rows of f32 in shared memory); 128 threads -------------

// out[d][off0 + m ldo + n0 + c] = bf16(tile[m][c]) into every destination
__device__ __forceinline__ void finish_bf16(const SegGemmArgs& a, const SegGemm& g, const float* tile, int n0, int valid, int te) {
    const bool vec = ((a.off0 + n0) & 7) == 0 && (a.ldo & 7) == 0 && (valid & 7) == 0;
    if (vec) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = te + 128 * i, m = idx >> 4, c8 = (idx & 15) * 8;
            if (m < g.M && c8 < valid) {
                const uint4 v = pack8f(tile + m * kTileLd + c8);
                for (int d = 0; d < a.n_out; ++d) *(uint4*)(a.out[d] + a.off0 + (long long)m * a.ldo + n0 + c8) = v;
            }
        }
    } else {
        for (int idx = te; idx < 16 * 128; idx += 128) {
            const int m = idx >> 7, c = idx & 127;
            if (m < g.M && c < valid) {
                const bf16 v = __float2bfloat16_rn(tile[m * kTileLd + c]);
                for (int d = 0; d < a.n_out; ++d) a.out[d][a.off0 + (long long)m * a.ldo + n0 + c] = v;
            }
        }
    }
}

// the same in f32 (the lm_head's gathered logits)
__device__ __forceinline__ void finish_f32(const SegGemmArgs& a, const SegGemm& g, const float* tile, int n0, int valid, int te) {
    const bool vec = ((a.off0 + n0) & 3) == 0 && (a.ldo & 3) == 0 && (valid & 3) == 0;
    if (vec) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = te + 128 * i, m = idx >> 5, c4 = (idx & 31) * 4;
            if (m < g.M && c4 < valid) {
                const float4 v = *(const float4*)(tile + m * kTileLd + c4);
                for (int d = 0; d < a.n_out; ++d) *(float4*)((float*)a.out[d] + a.off0 + (long long)m * a.ldo + n0 + c4) = v;
            }
        }
    } else {
        for (int idx = te; idx < 16 * 128; idx += 128) {
            const int m = idx >> 7, c = idx & 127;
            if (m < g.M && c < valid) {
                const float v = tile[m * kTileLd + c];
                for (int d = 0; d < a.n_out; ++d) ((float*)a.out[d])[a.off0 + (long long)m * a.ldo + n0 + c] = v;
            }
        }
    }
}

// the router: f32 logits and the routing's selection scores (sigmoid in f64 rounded to f32, plus the expert's bias)
__device__ __forceinline__ void finish_router(const SegGemmArgs& a, const SegGemm& g, const float* tile, int n0, int valid, int te) {
    for (int idx = te; idx < 16 * 128; idx += 128) {
        const int m = idx >> 7, c = idx & 127;
        if (m < g.M && c < valid) {
            const float v = tile[m * kTileLd + c];
            const int i = m * g.N + n0 + c;
            a.f32_out[i] = v;
            if (a.score != nullptr) a.score[i] = (float)(1.0 / (1.0 + exp(-((double)v * a.score_mult)))) + a.score_bias[n0 + c];
        }
    }
}

// the qkv head's row work, a warp per (row, 64-wide head): bf16(acc), per-head qk norm (q scaled), interleaved-pair RoPE, K
// and V rows appended to the successor's pool (arithmetic of test/reference/muse_spark.py:601-635)
__device__ __forceinline__ void finish_qkv(const SegGemmArgs& a, const SegGemm& g, const float* tile, int n0, int q, int lane) {
    const GemmArgs& e = a.epi;
    for (int it = q; it < g.M * 2; it += 4) {
        const int m = it >> 1, hl = it & 1, head = (n0 >> 6) + hl;
        if (head * kHeadDim >= g.N) continue;
        float y0 = bf16_round(tile[m * kTileLd + hl * 64 + 2 * lane]), y1 = bf16_round(tile[m * kTileLd + hl * 64 + 2 * lane + 1]);
        bf16* orow = (bf16*)e.out[0] + (size_t)m * e.ldo + head * kHeadDim + 2 * lane;
        const size_t slot_off = (size_t)e.cache_loc[m] * e.kv_row_bytes;
        if (head < e.qh + e.kvh) {
            const float ms = warp_sum(y0 * y0 + y1 * y1) * (1.0f / 64.0f);
            const float scale = (head < e.qh ? e.q_scale : 1.0f) * (1.0f / sqrtf(ms + e.eps));
            y0 = bf16_round(y0 * scale);
            y1 = bf16_round(y1 * scale);
            if (e.cos_sin) {
                const float c = e.cos_sin[m * 64 + lane], s = e.cos_sin[m * 64 + 32 + lane];
                const float r0 = fmaf(y0, c, -(y1 * s)), r1 = fmaf(y1, c, y0 * s);
                y0 = r0;
                y1 = r1;
            }
        }
        const __nv_bfloat162 o2 = __floats2bfloat162_rn(y0, y1);
        *(__nv_bfloat162*)orow = o2;
        if (head >= e.qh && head < e.qh + e.kvh && e.k_cache)
            *(__nv_bfloat162*)(e.k_cache + slot_off + (head - e.qh) * 128 + 4 * lane) = o2;
        if (head >= e.qh + e.kvh && head < e.qh + 2 * e.kvh && e.v_cache)
            *(__nv_bfloat162*)(e.v_cache + slot_off + (head - e.qh - e.kvh) * 128 + 4 * lane) = o2;
    }
}

// SwiGLU: the image pairs 64 gate rows (tile rows 0..63) with the same features' up rows (64..127):
// out[m, 64 tile + j] = bf16(silu(bf16(gate)) x bf16(up)), f32 steps in the order gate / (1 + exp(-gate)) x up
__device__ __forceinline__ void finish_silu(const SegGemmArgs& a, const SegGemm& g, const float* tile, int t, int te) {
    for (int idx = te; idx < 16 * 64; idx += 128) {
        const int m = idx >> 6, j = idx & 63;
        if (m >= g.M) continue;
        const float gate = bf16_round(tile[m * kTileLd + j]), up = bf16_round(tile[m * kTileLd + 64 + j]);
        const bf16 b = __float2bfloat16_rn(__fmul_rn(__fdiv_rn(gate, __fadd_rn(1.0f, expf(-gate))), up));
        for (int d = 0; d < a.n_out; ++d) a.out[d][a.off0 + (long long)m * a.ldo + t * 64 + j] = b;
    }
}

// A conv projection: the image holds, per tile, 32 groups' coefficients of the four (side, tap) kinds (tile row
// kind 32 + group). bf16 coefficients to c_out[m, kind groups + group], then the conv's side 0 over the rows the projection
// was computed from, a thread per (row, group), as segments.cuh seg_finish_conv.
__device__ __forceinline__ void finish_conv(const SegGemmArgs& a, const SegGemm& g, const float* tile, int t, int te) {
    const SegConv& cv = a.conv;
    const int gl0 = t * 32;
    for (int idx = te; idx < 16 * 128; idx += 128) {
        const int m = idx >> 7, r = idx & 127, kind = r >> 5, gi = gl0 + (r & 31);
        if (m < g.M && gi < cv.groups) a.out[0][(long long)m * a.ldo + kind * cv.groups + gi] = __float2bfloat16_rn(tile[m * kTileLd + r]);
    }
    const int per_group = cv.H / cv.groups;
    for (int idx = te; idx < 16 * 32; idx += 128) {
        const int m = idx >> 5, gl = idx & 31, gi = gl0 + gl;
        if (m >= g.M || gi >= cv.groups) continue;
        const float d0 = bf16_round(tile[m * kTileLd + gl]), d1 = bf16_round(tile[m * kTileLd + 32 + gl]);
        for (int c0 = gi * per_group; c0 < (gi + 1) * per_group; c0 += 8) {
            float b0[8], b1[8], x[8], xp[8], out[8];
            load8(cv.base + c0, b0);
            load8(cv.h + (size_t)m * cv.H + c0, x);
            if (m > 0) {
                load8(cv.base + cv.H + c0, b1);
                load8(cv.h + (size_t)(m - 1) * cv.H + c0, xp);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                out[j] = __fmul_rn(__fadd_rn(b0[j], d0), x[j]);
                if (m > 0) out[j] = __fadd_rn(out[j], __fmul_rn(__fadd_rn(b1[j], d1), xp[j]));
            }
            store8(cv.xa + (size_t)m * cv.H + c0, out);
        }
    }
}

// The draft's qkv: a tile is one 128-wide head; a warp per row rounds it to bf16 (the stored qkv row), then head norm, neox
// RoPE and the K / V append (draft_rows.cuh dqkv_head).
__device__ __forceinline__ void finish_dqkv(const SegGemmArgs& a, const SegGemm& g, const float* tile, int t, int q, int lane) {
    const DQkvRowsArgs& r = a.rows;
    const long long P = r.words[kWordP];
    for (int m = q; m < g.M; m += 4) {
        const float* row = tile + m * kTileLd;
        const __nv_bfloat162 ql = __floats2bfloat162_rn(row[2 * lane], row[2 * lane + 1]);
        const __nv_bfloat162 qh = __floats2bfloat162_rn(row[64 + 2 * lane], row[64 + 2 * lane + 1]);
        bf16* orow = a.out[0] + (long long)m * a.ldo + t * kDraftHeadDim;
        *(__nv_bfloat162*)(orow + 2 * lane) = ql;
        *(__nv_bfloat162*)(orow + 64 + 2 * lane) = qh;
        float v[4] = {__low2float(ql), __high2float(ql), __low2float(qh), __high2float(qh)};
        dqkv_head(r, m, t, v, P, lane);
    }
}


// ---- the engine's shared memory and per-CTA context ----------------------------------------------------------------------------
template <int RING>
struct DenseLayout {
    static constexpr size_t kRingBytes = (size_t)RING * (kStageW + kStageX);
    static constexpr size_t kTileBytes = 16 * kTileLd * 4;
    static constexpr size_t kBarBytes = (3 * RING + 4) * 8 + 16;
    static constexpr size_t kBytes = 1024 + kRingBytes + kTileBytes + kBarBytes;  // then the caller's own scratch
};

struct DenseCtx {
    unsigned char* wring;
    unsigned char* xring;
    float* tile;
    uint64_t* full_w;
    uint64_t* full_x;
    uint64_t* empty;
    uint64_t* acc_full;   // [2]
    uint64_t* acc_empty;  // [2]
    uint32_t* tmem_slot;
    volatile int* abort;
    volatile int* is_last;
    unsigned char* extra;  // first byte behind the engine's shared memory
    uint32_t tmem;
    int* status;
    int trace_id;  // trace builds: the launch's row of the trace array (-1: none)
};

// Carves the dynamic shared memory, initialises the barriers and allocates the tensor memory; ends with a block-wide
// barrier. Every thread of the CTA calls it.
template <int RING>
__device__ __forceinline__ DenseCtx dense_setup_cta(unsigned char* raw, int* status) {
    DenseCtx c;
    unsigned char* smem = (unsigned char*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    c.wring = smem;
    c.xring = smem + RING * kStageW;
    c.tile = (float*)(c.xring + RING * kStageX);
    uint64_t* bars = (uint64_t*)(c.tile + 16 * kTileLd);
    c.full_w = bars;
    c.full_x = bars + RING;
    c.empty = bars + 2 * RING;
    c.acc_full = bars + 3 * RING;
    c.acc_empty = bars + 3 * RING + 2;
    c.tmem_slot = (uint32_t*)(bars + 3 * RING + 4);
    c.abort = (volatile int*)(c.tmem_slot + 1);
    c.is_last = (volatile int*)(c.tmem_slot + 2);
    c.extra = (unsigned char*)bars + DenseLayout<RING>::kBarBytes;
    c.status = status;
    c.trace_id = -1;
    if (threadIdx.x == 0) {
        for (int i = 0; i < RING; ++i) {
            mbar_init(&c.full_w[i], 1);
            mbar_init(&c.full_x[i], 64);
            mbar_init(&c.empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&c.acc_full[i], 1);
            mbar_init(&c.acc_empty[i], 128);
        }
        *c.abort = 0;
        mbar_fence_init();
    }
    if ((threadIdx.x >> 5) == 2) tmem_alloc(c.tmem_slot, kDTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    c.tmem = *c.tmem_slot;
    return c;
}
// Every thread of the CTA, after all roles are done.
__device__ __forceinline__ void dense_teardown_cta(const DenseCtx& c) {
    tc_fence_before();
    __syncthreads();
    if ((threadIdx.x >> 5) == 2) tmem_dealloc(c.tmem, kDTmemCols);
}

// ---- roles -------------------------------------------------------------------------------------------------------------------
// Each runs this CTA's units of one GEMM stage and keeps its counters (ring position `it`, accumulator index `i`) for the
// next stage of the same kernel. All return false once the CTA's abort flag is up.

// warp 0 lane 0: streams the weight stages. No dependency on anything the GPU computes.
template <int RING>
__device__ __forceinline__ bool dense_produce(const SegGemmArgs& a, const DenseCtx& c, const Plan& pl, uint32_t& it, uint64_t policy) {
    for (uint32_t p = pl.lo; p < pl.hi;) {
        if (*c.abort) return false;
        const Unit u = unit_at(a, pl, p);
        const SegGemm& g = a.g[u.gi];
        const int KS = stages_of(g), valid = min(128, g.N - u.tile * 128);
        const uint32_t bytes = (uint32_t)((valid + 7) & ~7) * 128u;
        const unsigned char* src = g.w + ((size_t)u.tile * KS + u.k0) * kStageW;
        for (int ks = u.k0; ks < u.k1; ++ks, ++it, src += kStageW) {
            const uint32_t s = it % RING, round = it / RING;
            if (!mbar_wait(&c.empty[s], (round & 1) ^ 1, c.abort)) {
                dense_abort(c.status, c.abort, 500, (int)it);
                return false;
            }
            mbar_arrive_expect_tx(&c.full_w[s], 2 * bytes);
            unsigned char* dst = c.wring + s * kStageW;
            bulk_g2s_hint(dst, src, bytes, &c.full_w[s], policy);
            bulk_g2s_hint(dst + kAtomW, src + kAtomW, bytes, &c.full_w[s], policy);
        }
        p += u.k1 - u.k0;
    }
    DT(2)
    return true;
}

// warp 1 lane 0: issues the MMAs of every stage as its weights and activations land.
template <int RING>
__device__ __forceinline__ bool dense_mma(const SegGemmArgs& a, const DenseCtx& c, const Plan& pl, uint32_t& it, int& i) {
    for (uint32_t p = pl.lo; p < pl.hi; ++i) {
        if (*c.abort) return false;
        const Unit u = unit_at(a, pl, p);
        const bool tf32 = a.g[u.gi].f32 != 0;
        const int buf = i & 1;
        if (!mbar_wait(&c.acc_empty[buf], ((i >> 1) & 1) ^ 1, c.abort)) {
            dense_abort(c.status, c.abort, 510, i);
            return false;
        }
        tc_fence_after();
        const uint32_t d = c.tmem + buf * 16;
        for (int ks = u.k0; ks < u.k1; ++ks, ++it) {
            const uint32_t s = it % RING, round = it / RING;
            if (!mbar_wait(&c.full_w[s], round & 1, c.abort) || !mbar_wait(&c.full_x[s], round & 1, c.abort)) {
                dense_abort(c.status, c.abort, 520, (int)it);
                return false;
            }
            tc_fence_after();
            if (p == pl.lo && ks == u.k0) { DT(5) }
            const uint32_t wb = smem_u32(c.wring + s * kStageW), xb = smem_u32(c.xring + s * kStageX);
#pragma unroll
            for (int at = 0; at < 2; ++at)
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint64_t ad = desc_sw128(wb + at * kAtomW + kk * 32), bd = desc_sw128(xb + at * kAtomX + kk * 32);
                    const uint32_t acc = (ks != u.k0 || at != 0 || kk != 0) ? 1u : 0u;
                    if (tf32) mma_tf32(d, ad, bd, acc);
                    else mma_bf16(d, ad, bd, acc);
                }
            tc_commit(&c.empty[s]);
        }
        tc_commit(&c.acc_full[buf]);
        DT(6)
        p += u.k1 - u.k0;
    }
    return true;
}

// warps 2-3 (ts = 0..63): the window's rows of every stage into the swizzled B layout, kXDepth stages in flight per
// thread. The stage's last copies are waited for before returning: nothing of this GEMM stage is left pending when the
// caller goes on to wait for the next stage's inputs.
template <int RING>
__device__ __forceinline__ bool dense_stage_x(const SegGemmArgs& a, const DenseCtx& c, const Plan& pl, uint32_t& it, int ts) {
    uint32_t arrived = it;
    const uint32_t it0 = it;
    bool ok = true;
    for (uint32_t p = pl.lo; p < pl.hi && ok;) {
        const Unit u = unit_at(a, pl, p);
        const SegGemm& g = a.g[u.gi];
        for (int ks = u.k0; ks < u.k1; ++ks, ++it) {
            const uint32_t s = it % RING, round = it / RING;
            ok = mbar_wait(&c.empty[s], (round & 1) ^ 1, c.abort);
            if (!ok) {
                dense_abort(c.status, c.abort, 530, (int)it);
                break;
            }
            unsigned char* dst = c.xring + s * kStageX;
            const unsigned char* src = g.x + (size_t)ks * 256;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int idx = k * 64 + ts, m = idx >> 4, at = (idx >> 3) & 1, j = idx & 7;
                if (m < g.M)
                    cp_async16(dst + at * kAtomX + (m >> 3) * 1024 + (m & 7) * 128 + ((j ^ (m & 7)) << 4),
                               src + (size_t)m * g.ldx + at * 128 + j * 16, true);
            }
            cp_async_commit();
            if (it - it0 + 1 >= (uint32_t)kXDepth) {  // the stage issued kXDepth - 1 iterations ago has landed
                cp_async_wait<kXDepth - 1>();
                fence_proxy_async_smem();
                mbar_arrive(&c.full_x[arrived % RING]);
                if (arrived == it0 && ts == 0) { DT(4) }
                ++arrived;
            }
        }
        p += u.k1 - u.k0;
    }
    cp_async_wait<0>();
    fence_proxy_async_smem();
    if (ok)
        for (; arrived < it; ++arrived) mbar_arrive(&c.full_x[arrived % RING]);
    return ok;
}

// What the epilogue does for the world once a tile is finished (all null / zero: nothing): `tile_sig[gi]` the exchange the
// tile's peer stores feed (one arrival per finished tile on every receiving rank), `dep[gi]` a device counter that CTAs of
// this kernel wait on.
struct TileSignals {
    const XchgSignal* tile_sig[2];
    unsigned* dep[2];
    bool defer1;  // the second GEMM's tiles are not finished here: every contributor stores its partial and arrives on
                  // dep[1]; whoever waits for all contributions sums them in slot order (the router's rows, fused.cuh)
};

// warps 4-7 (te = 0..127, q = warp - 4): accumulators out of tensor memory, the stream-K meeting of a shared tile, the
// epilogue of a finished one.
template <int RING>
__device__ __forceinline__ bool dense_epilogue(const SegGemmArgs& a, const DenseCtx& c, const Plan& pl, int& i, int q, int te, int lane,
                                               const TileSignals& sg) {
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    float* tile = c.tile;
    for (uint32_t p = pl.lo; p < pl.hi; ++i) {
        const Unit u = unit_at(a, pl, p);
        const SegGemm& g = a.g[u.gi];
        const int buf = i & 1;
        if (!bar_all(2, 128, mbar_wait(&c.acc_full[buf], (i >> 1) & 1, c.abort))) {
            if (te == 0) dense_abort(c.status, c.abort, 540, i);
            return false;
        }
        tc_fence_after();
        if (p == pl.lo && te == 0) { DT(7) }
        uint32_t r[16];
        tmem_ld16(c.tmem + lane_base + buf * 16, r);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&c.acc_empty[buf]);
        float v[16];
#pragma unroll
        for (int m = 0; m < 16; ++m) v[m] = __uint_as_float(r[m]);
        bool finish = true;
        if (u.gi == 1 && sg.defer1) {
            float* mine = g.part + ((size_t)u.tile * g.maxc + u.slot) * 2048 + te;
#pragma unroll
            for (int m = 0; m < 16; ++m) __stcg(mine + m * 128, v[m]);
            __threadfence();
            bar_sync(2, 128);
            if (te == 0) atomicAdd(sg.dep[1], 1u);
            finish = false;
        } else if (u.n > 1) {
            // this CTA's partial of the tile, then a ticket: the last contributor sums all of them in slot order
            float* mine = g.part + ((size_t)u.tile * g.maxc + u.slot) * 2048 + te;
#pragma unroll
            for (int m = 0; m < 16; ++m) __stcg(mine + m * 128, v[m]);
            __threadfence();
            bar_sync(2, 128);
            if (te == 0) *c.is_last = atomicInc(g.ticket + u.tile, (unsigned)(u.n - 1)) == (unsigned)(u.n - 1);
            bar_sync(2, 128);
            finish = *c.is_last != 0;
            if (finish) {
                __threadfence();
#pragma unroll
                for (int m = 0; m < 16; ++m) v[m] = 0.f;
                // four contributors' partials are requested before the first is added: the sum's order stays slot order
                for (int sl = 0; sl < u.n; sl += 4) {
                    float t[4][16];
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        if (sl + k < u.n) {
                            const float* src = g.part + ((size_t)u.tile * g.maxc + sl + k) * 2048 + te;
#pragma unroll
                            for (int m = 0; m < 16; ++m) t[k][m] = __ldcg(src + m * 128);
                        }
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        if (sl + k < u.n) {
#pragma unroll
                            for (int m = 0; m < 16; ++m) v[m] += t[k][m];
                        }
                }
            }
        }
        if (finish) {
            if (te == 0) { DT(10) }
#pragma unroll
            for (int m = 0; m < 16; ++m) tile[m * kTileLd + te] = v[m];
            bar_sync(2, 128);
            const int n0 = u.tile * 128, valid = min(128, g.N - n0);
            if (u.gi == 1) finish_router(a, g, tile, n0, valid, te);
            else if (a.finish == 2) finish_qkv(a, g, tile, n0, q, lane);
            else if (a.finish == 3) finish_silu(a, g, tile, u.tile, te);
            else if (a.finish == 4) finish_f32(a, g, tile, n0, valid, te);
            else if (a.finish == 5) finish_conv(a, g, tile, u.tile, te);
            else if (a.finish == 6) finish_dqkv(a, g, tile, u.tile, q, lane);
            else finish_bf16(a, g, tile, n0, valid, te);
            const XchgSignal* xs = sg.tile_sig[u.gi];
            unsigned* dep = sg.dep[u.gi];
            if ((xs != nullptr && xs->n > 0) || dep != nullptr) {
                // the tile's stores, then one arrival: device scope for waiters on this GPU, system scope for peers
                const bool remote = xs != nullptr && xs->n > 0 && xs->remote;
                if (remote) __threadfence_system();
                else __threadfence();
                bar_sync(2, 128);
                if (te == 0) {
                    if (xs != nullptr)
                        for (int r2 = 0; r2 < xs->n; ++r2) {
                            if (xs->remote) atomicAdd_system(xs->flag[r2], 1u);
                            else atomicAdd(xs->flag[r2], 1u);
                        }
                    if (dep != nullptr) atomicAdd(dep, 1u);
                }
            }
        }
        bar_sync(2, 128);  // the tile and the ticket flag are free again
        p += u.k1 - u.k0;
    }
    if (te == 0) { DT(8) }
    return true;
}

}  // namespace mk
