// The dense GEMMs of the decode path (o_proj, pooler, router, unpooler, qkv head, lm_head, the draft's projections) on the
// 5th-generation tensor cores: out[m, n] = sum_k x[m, k] W[n, k] with at most 16 activation rows.
//
// Shape of the contraction ("swap-AB"): the WEIGHTS are the M = 128 operand of tcgen05.mma (kind::f16 for bf16 weights,
// kind::tf32 for the f32 router), the window's rows the N = 16 operand, the accumulator a [128 lanes x 16 columns] f32 block
// of tensor memory. The accumulation over K never leaves tensor memory while a CTA works on a tile.
//
// Work split ("stream-K"): a GEMM is tiles x K-stages stage units, a stage unit being 128 weight rows x 256 bytes of K
// (128 bf16 or 64 f32 elements: two 128-byte-swizzle atoms). The stage units of the launch's one or two GEMMs form one
// sequence that is cut into equal contiguous ranges, one per CTA, whatever the shape: every CTA streams the same number of
// bytes. A tile whose K range is shared by several CTAs is finished by the last of them to arrive: each writes its [16 x 128]
// f32 partial to L2-resident scratch, takes a ticket (atomicInc that wraps at the number of contributors, so the word is
// back at zero for the next launch), and the holder of the last ticket sums the partials in contributor order (a fixed
// order: results do not depend on timing) and runs the epilogue. There is no grid barrier and no second pass.
//
// Weight image (built once by the host, sgl_muse_mega_b200/muse_spark/b200/weights.py pack_umma): for every
// (tile, K stage) 32 KiB: atom 0 then atom 1, an atom = 128 rows x 128 bytes with the 16-byte chunk j of row r stored at
// chunk j ^ (r % 8) (the K-major 128-byte-swizzle operand layout); rows past N are zero. One stage arrives by two bulk
// copies (only the valid rows of a ragged last tile are read). The router's image has the low 13 mantissa bits cleared.
//
// Roles (256 threads): warp 0 lane 0 streams weight stages through a 6-deep ring (starting before the programmatic
// launch wait: weights do not depend on the predecessor), warps 2-3 copy the activation slice of every stage into the
// swizzled B layout with cp.async (three stages in flight per thread), warp 1 lane 0 issues the MMAs, warps 4-7 read the
// accumulators and run the epilogue (bf16 / f32 stores into every destination, router scores, the qkv row work, SwiGLU,
// the draft's conv and head work). Two accumulators alternate, so the MMAs of a CTA's next tile run under the epilogue
// of the previous one.
//
// Every wait is bounded: an expired wait raises the CTA's abort flag, records itself in the launch's status block (code 3)
// and every role leaves through the common teardown, which releases the tensor memory. Nothing traps.
//
// Reference counterparts: sm103/kernels/framework.cuh:349-706 (dense_body: kind::f16 tiles, TMEM accumulators, TMA ring,
// weights before griddepcontrol.wait), kernels/ptx.cuh:872-880 (kind::tf32 router).
#include "draft_rows.cuh"
#include "umma.cuh"

namespace mk {

using namespace umma;

namespace {

constexpr int kDThreads = 256;
constexpr uint32_t kAtomW = 128 * 128;   // 128 weight rows x 128 bytes
constexpr uint32_t kStageW = 2 * kAtomW;
constexpr uint32_t kAtomX = 16 * 128;    // 16 window rows x 128 bytes
constexpr uint32_t kStageX = 2 * kAtomX;
constexpr int kRing = 6;
constexpr int kTileLd = 132;             // floats per row of the epilogue tile (16 rows x 128 columns, padded)
constexpr uint32_t kDTmemCols = 32;      // two accumulators of 16 columns
constexpr int kXDepth = 3;               // activation stages a stager thread keeps in flight
constexpr int kDenseMaxGrid = 148;

struct Unit {
    int gi, tile, k0, k1, slot, n;
};

__device__ __forceinline__ int stages_of(const SegGemm& g) { return g.K * (g.f32 ? 4 : 2) / 256; }
__device__ __forceinline__ int tiles_of(const SegGemm& g) { return (g.N + 127) / 128; }

// the CTA whose range holds stage unit s: the largest c with floor(c T / G) <= s
__device__ __forceinline__ int cta_of(long long s, long long T, long long G) { return (int)(((s + 1) * G + T - 1) / T - 1); }

__device__ __forceinline__ Unit unit_at(const SegGemmArgs& a, long long T0, long long T, long long G, long long p, long long hi) {
    Unit u;
    u.gi = p >= T0 ? 1 : 0;
    const long long base = u.gi ? T0 : 0;
    const int KS = stages_of(a.g[u.gi]);
    const long long rel = p - base;
    u.tile = (int)(rel / KS);
    u.k0 = (int)(rel - (long long)u.tile * KS);
    const long long left = hi - p;
    u.k1 = (int)(left < KS - u.k0 ? u.k0 + left : KS);
    const long long first = base + (long long)u.tile * KS;
    const int c0 = cta_of(first, T, G), c1 = cta_of(first + KS - 1, T, G);
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

// weights are read once: evict-first in L2, so that the activations, partial sums and exchange buffers stay resident
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void bulk_g2s_hint(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
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

}  // namespace

// Trace builds (-DDENSE_TRACE): the first, middle and last CTA stamp the global timer (ns) into u64 words [32 + 16 w + slot]
// of the launch's status block (w = 0, 1, 2): 0 kernel entry, 1 set-up done, 2 first weight copy issued, 3 first stage
// landed (MMA thread), 4 last MMA issued, 5 first accumulator complete (epilogue), 6 partial stored and ticket taken,
// 7 epilogue done, 8 teardown, 9 first activation stage landed.
#ifdef DENSE_TRACE
#define DT(slot)                                                                                                   \
    if (a.status != nullptr && (blockIdx.x == 0 || blockIdx.x == gridDim.x / 2 || blockIdx.x == gridDim.x - 1)) { \
        unsigned long long t_;                                                                                     \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                                    \
        const int w_ = blockIdx.x == 0 ? 0 : (blockIdx.x == gridDim.x - 1 ? 2 : 1);                                \
        ((unsigned long long*)a.status)[32 + 16 * w_ + (slot)] = t_;                                               \
    }
#else
#define DT(slot)
#endif

__global__ void __launch_bounds__(kDThreads, 1) dense_umma_kernel(const SegGemmArgs a) {
    extern __shared__ unsigned char dense_smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)dense_smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* wring = smem;
    unsigned char* xring = smem + kRing * kStageW;
    float* tile = (float*)(xring + kRing * kStageX);
    uint64_t* bars = (uint64_t*)(tile + 16 * kTileLd);
    uint64_t* full_w = bars;
    uint64_t* full_x = bars + kRing;
    uint64_t* empty = bars + 2 * kRing;
    uint64_t* acc_full = bars + 3 * kRing;       // [2]
    uint64_t* acc_empty = bars + 3 * kRing + 2;  // [2]
    uint32_t* tmem_slot = (uint32_t*)(bars + 3 * kRing + 4);
    volatile int* abort = (volatile int*)(tmem_slot + 1);
    volatile int* is_last = (volatile int*)(tmem_slot + 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        DT(0)
        for (int i = 0; i < kRing; ++i) {
            mbar_init(&full_w[i], 1);
            mbar_init(&full_x[i], 64);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 128);
        }
        *abort = 0;
        mbar_fence_init();
    }
    if (warp == 2) tmem_alloc(tmem_slot, kDTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    if (tid == 0) { DT(1) }

    // this CTA's range of the launch's stage units
    const long long T0 = (long long)tiles_of(a.g[0]) * stages_of(a.g[0]);
    const long long T = T0 + (a.n_gemm > 1 ? (long long)tiles_of(a.g[1]) * stages_of(a.g[1]) : 0);
    const long long G = gridDim.x;
    const long long lo = (long long)blockIdx.x * T / G, hi = (long long)(blockIdx.x + 1) * T / G;

    if (warp == 0) {
        // ---- weight producer: no dependency on the predecessor, starts at once ----
        if (lane == 0) {
            const uint64_t policy = policy_evict_first();
            uint32_t it = 0;
            for (long long p = lo; p < hi && !*abort;) {
                const Unit u = unit_at(a, T0, T, G, p, hi);
                const SegGemm& g = a.g[u.gi];
                const int KS = stages_of(g), valid = min(128, g.N - u.tile * 128);
                const uint32_t bytes = (uint32_t)((valid + 7) & ~7) * 128u;
                const unsigned char* src = g.w + ((size_t)u.tile * KS + u.k0) * kStageW;
                bool ok = true;
                for (int ks = u.k0; ks < u.k1; ++ks, ++it, src += kStageW) {
                    const uint32_t s = it % kRing, round = it / kRing;
                    if (!mbar_wait(&empty[s], (round & 1) ^ 1, abort)) {
                        dense_abort(a.status, abort, 500, (int)it);
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&full_w[s], 2 * bytes);
                    unsigned char* dst = wring + s * kStageW;
                    bulk_g2s_hint(dst, src, bytes, &full_w[s], policy);
                    bulk_g2s_hint(dst + kAtomW, src + kAtomW, bytes, &full_w[s], policy);
                    if (it == 0) { DT(2) }
                }
                if (!ok) break;
                p += u.k1 - u.k0;
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue ----
        if (lane == 0) {
            uint32_t it = 0;
            int i = 0;
            for (long long p = lo; p < hi && !*abort; ++i) {
                const Unit u = unit_at(a, T0, T, G, p, hi);
                const bool tf32 = a.g[u.gi].f32 != 0;
                const int buf = i & 1;
                if (!mbar_wait(&acc_empty[buf], ((i >> 1) & 1) ^ 1, abort)) {
                    dense_abort(a.status, abort, 510, i);
                    break;
                }
                tc_fence_after();
                const uint32_t d = tmem + buf * 16;
                bool ok = true;
                for (int ks = u.k0; ks < u.k1; ++ks, ++it) {
                    const uint32_t s = it % kRing, round = it / kRing;
                    if (!mbar_wait(&full_w[s], round & 1, abort) || !mbar_wait(&full_x[s], round & 1, abort)) {
                        dense_abort(a.status, abort, 520, (int)it);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    if (it == 0) { DT(3) }
                    const uint32_t wb = smem_u32(wring + s * kStageW), xb = smem_u32(xring + s * kStageX);
#pragma unroll
                    for (int at = 0; at < 2; ++at)
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const uint64_t ad = desc_sw128(wb + at * kAtomW + kk * 32), bd = desc_sw128(xb + at * kAtomX + kk * 32);
                            const uint32_t acc = (ks != u.k0 || at != 0 || kk != 0) ? 1u : 0u;
                            if (tf32) mma_tf32(d, ad, bd, acc);
                            else mma_bf16(d, ad, bd, acc);
                        }
                    tc_commit(&empty[s]);
                }
                if (!ok) break;
                tc_commit(&acc_full[buf]);
                DT(4)
                p += u.k1 - u.k0;
            }
        }
    } else if (warp < 4) {
        // ---- activation stager: the window's rows of every stage into the swizzled B layout ----
        griddep_wait();
        const int ts = tid - 64;  // 0..63
        uint32_t it = 0, arrived = 0;
        bool ok = true;
        for (long long p = lo; p < hi && ok;) {
            const Unit u = unit_at(a, T0, T, G, p, hi);
            const SegGemm& g = a.g[u.gi];
            for (int ks = u.k0; ks < u.k1; ++ks, ++it) {
                const uint32_t s = it % kRing, round = it / kRing;
                ok = mbar_wait(&empty[s], (round & 1) ^ 1, abort);
                if (!ok) {
                    dense_abort(a.status, abort, 530, (int)it);
                    break;
                }
                unsigned char* dst = xring + s * kStageX;
                const unsigned char* src = g.x + (size_t)ks * 256;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int idx = k * 64 + ts, m = idx >> 4, at = (idx >> 3) & 1, j = idx & 7;
                    if (m < g.M)
                        cp_async16(dst + at * kAtomX + (m >> 3) * 1024 + (m & 7) * 128 + ((j ^ (m & 7)) << 4),
                                   src + (size_t)m * g.ldx + at * 128 + j * 16, true);
                }
                cp_async_commit();
                if (it + 1 >= (uint32_t)kXDepth) {  // the stage issued kXDepth - 1 iterations ago has landed
                    cp_async_wait<kXDepth - 1>();
                    fence_proxy_async_smem();
                    mbar_arrive(&full_x[arrived % kRing]);
                    if (arrived == 0 && ts == 0) { DT(9) }
                    ++arrived;
                }
            }
            p += u.k1 - u.k0;
        }
        cp_async_wait<0>();
        fence_proxy_async_smem();
        if (ok)
            for (; arrived < it; ++arrived) mbar_arrive(&full_x[arrived % kRing]);
    } else {
        // ---- epilogue ----
        griddep_wait();
        const int q = warp - 4, te = tid - 128;
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        int i = 0;
        for (long long p = lo; p < hi; ++i) {
            const Unit u = unit_at(a, T0, T, G, p, hi);
            const SegGemm& g = a.g[u.gi];
            const int buf = i & 1;
            if (!bar_all(2, 128, mbar_wait(&acc_full[buf], (i >> 1) & 1, abort))) {
                if (te == 0) dense_abort(a.status, abort, 540, i);
                break;
            }
            tc_fence_after();
            if (i == 0 && te == 0) { DT(5) }
            uint32_t r[16];
            tmem_ld16(tmem + lane_base + buf * 16, r);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(&acc_empty[buf]);
            float v[16];
#pragma unroll
            for (int m = 0; m < 16; ++m) v[m] = __uint_as_float(r[m]);
            bool finish = true;
            if (u.n > 1) {
                // this CTA's partial of the tile, then a ticket: the last contributor sums all of them in slot order
                float* mine = g.part + ((size_t)u.tile * g.maxc + u.slot) * 2048 + te;
#pragma unroll
                for (int m = 0; m < 16; ++m) __stcg(mine + m * 128, v[m]);
                __threadfence();
                bar_sync(2, 128);
                if (te == 0) *is_last = atomicInc(g.ticket + u.tile, (unsigned)(u.n - 1)) == (unsigned)(u.n - 1);
                bar_sync(2, 128);
                if (te == 0) { DT(6) }
                finish = *is_last != 0;
                if (finish) {
                    __threadfence();
#pragma unroll
                    for (int m = 0; m < 16; ++m) v[m] = 0.f;
                    for (int sl = 0; sl < u.n; ++sl) {
                        const float* src = g.part + ((size_t)u.tile * g.maxc + sl) * 2048 + te;
#pragma unroll
                        for (int m = 0; m < 16; ++m) v[m] += __ldcg(src + m * 128);
                    }
                }
            }
            if (finish) {
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
            }
            bar_sync(2, 128);  // the tile and the ticket flag are free again
            if (te == 0) { DT(7) }
            p += u.k1 - u.k0;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2) tmem_dealloc(tmem, kDTmemCols);
    if (tid == 0) { DT(8) }
    xchg_signal(a.sig);
}

size_t dense_smem() { return 1024 + (size_t)kRing * (kStageW + kStageX) + 16 * kTileLd * 4 + (3 * kRing + 4) * 8 + 16; }

cudaError_t dense_prepare() {
    return cudaFuncSetAttribute(dense_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dense_smem());
}

static long long dense_units(const SegGemm& g) { return (long long)((g.N + 127) / 128) * (g.K * (g.f32 ? 4 : 2) / 256); }

int dense_grid(const SegGemmArgs& a, int sms) {
    long long T = dense_units(a.g[0]) + (a.n_gemm > 1 ? dense_units(a.g[1]) : 0);
    long long G = sms < kDenseMaxGrid ? sms : kDenseMaxGrid;
    if (T < G) G = T;
    return (int)(G < 1 ? 1 : G);
}

size_t dense_part_bound(long long N) { return (size_t)(2 * kDenseMaxGrid + 2 * ((N + 127) / 128)) * 2048; }

// Carves the launch's partial-sum scratch and tickets; false when they do not fit or a shape is not whole stages.
bool dense_setup(SegGemmArgs& a, int sms, float* part, size_t part_floats, unsigned* ticket, size_t ticket_words) {
    for (int i = 0; i < a.n_gemm; ++i) {
        const SegGemm& g = a.g[i];
        if (g.N < 1 || g.M < 1 || g.M > 16 || g.K < 1 || (g.K * (g.f32 ? 4 : 2)) % 256 != 0) return false;
        if (((uintptr_t)g.w & 15) || ((uintptr_t)g.x & 15) || (g.ldx & 15)) return false;
    }
    const int G = dense_grid(a, sms);
    const long long T = dense_units(a.g[0]) + (a.n_gemm > 1 ? dense_units(a.g[1]) : 0);
    const long long per = T / G;  // >= 1
    size_t used = 0, tickets = 0;
    for (int i = 0; i < a.n_gemm; ++i) {
        SegGemm& g = a.g[i];
        const long long KS = g.K * (g.f32 ? 4 : 2) / 256, tiles = (g.N + 127) / 128;
        g.maxc = (int)((KS + per - 1) / per + 1);
        g.part = part + used;
        g.ticket = ticket + tickets;
        used += (size_t)tiles * g.maxc * 2048;
        tickets += (size_t)tiles;
    }
    return used <= part_floats && tickets <= ticket_words;
}

cudaError_t dense_launch(const SegGemmArgs& a, int sms, cudaStream_t s, bool pdl) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(dense_grid(a, sms));
    cfg.blockDim = dim3(kDThreads);
    cfg.dynamicSmemBytes = dense_smem();
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, dense_umma_kernel, a);
}

}  // namespace mk
