// The bf16 experts (the model's first and last layer) on the 5th-generation tensor cores: a grouped GEMM over the routed
// experts with the dense engine's pipeline (dense.cuh).
//
// For every routed expert e and every 128-row tile of its weight: out[slot, tile rows] = sum_k x[row of slot, k] W_e[row, k]
// over the <= 16 slots routed to e. The weights are the M = 128 operand of tcgen05.mma kind::f16, the expert's rows the
// N = 16 operand, the accumulator a [128 lanes x 16 columns] f32 block of tensor memory (two alternate).
//   g1: W_e = the expert's [gate | up] rows with each tile holding 64 gate rows and the same features' up rows
//       (weights.py silu_perm), x = the normed pooled rows by token; finish: z = bf16(silu(bf16(gate)) x bf16(up)) into
//       every peer's h rows [slot, rank I_s + feature].
//   g2: W_e = the expert's w2 rows, x = the gathered h rows by slot; finish: zb[slot, rank H_s + row] = bf16(acc) into every
//       peer's expert outputs.
// Arithmetic contract: test/reference/muse_spark.py:566-584.
//
// Weight image (weights.py pack_umma over the experts' rows): [E][tiles per expert][K bytes / 256] stages of 32 KiB (two
// 128-byte-swizzle K-major atoms), one stage = two 1-D bulk copies with an evict-first policy (expert weights are read once
// a step).
//
// Work split: the launch's (routed expert, tile) units x K stages form one sequence of weight stages that is cut into equal
// contiguous ranges, one per CTA (over min(grid, stages) CTAs), so every CTA streams the same number of bytes whatever the
// number of routed experts. At most the first and the last item of a CTA's range are pieces of a unit shared with the
// neighbouring CTAs: a piece's accumulators go to L2-resident scratch (two slots per CTA), its CTA takes a ticket
// (atomicInc that wraps at the number of contributors: the word is zero again for the next launch; the ticket of a unit
// is the word of the first CTA that holds a piece of it), and the holder of the last ticket sums the pieces in CTA order
// (a fixed order) and runs the finish. There is no wait between CTAs.
//
// Roles (256 threads, as the dense engine): warp 0 lane 0 streams weight stages through a 5-deep ring, warps 2-3 gather
// the unit's rows of every stage into the swizzled B layout with cp.async, warp 1 lane 0 issues the MMAs, warps 4-7 run
// the epilogue from tensor memory. Every wait is bounded; an expired wait raises the CTA's abort flag, records itself in
// the status block (code 3) and every role leaves through the common teardown, which releases the tensor memory.
#include "dense.cuh"

namespace mk {

namespace {

constexpr int kBRing = 5;

struct Item {
    int u, k0, k1, c0, n;
};
// the CTA whose range [floor(c T / G), floor((c + 1) T / G)) holds stage s
__device__ __forceinline__ int cta_holding(uint32_t s, uint32_t T, uint32_t G) { return (int)(((s + 1) * G + T - 1) / T - 1); }
__device__ __forceinline__ Item item_at(uint32_t p, uint32_t hi, uint32_t T, uint32_t G, uint32_t KS) {
    Item w;
    w.u = (int)(p / KS);
    w.k0 = (int)(p - (uint32_t)w.u * KS);
    const uint32_t left = hi - p;
    w.k1 = (int)(left < KS - (uint32_t)w.k0 ? (uint32_t)w.k0 + left : KS);
    const uint32_t first = (uint32_t)w.u * KS;
    w.c0 = cta_holding(first, T, G);
    w.n = cta_holding(first + KS - 1, T, G) - w.c0 + 1;
    return w;
}
// scratch slot of contributor c to a shared unit whose first contributor is c0: a CTA's range begins with at most one
// unit's tail piece (slot 2 c) and ends with at most one unit's head piece (slot 2 c + 1)
__device__ __forceinline__ size_t piece_slot(int c, int c0) { return (size_t)(2 * c + (c == c0 ? 1 : 0)); }

}  // namespace

__global__ void __launch_bounds__(kDThreads, 1) experts_bf16_umma_kernel(const __grid_constant__ Bf16UmmaArgs a) {
    extern __shared__ unsigned char bf16_smem_raw[];
    const DenseCtx c = dense_setup_cta<kBRing>(bf16_smem_raw, a.status);
    RouteTables* rt = (RouteTables*)(((uintptr_t)c.extra + 15) & ~(uintptr_t)15);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // g1 follows the routing kernel; g2's predecessor is g1 (the tables were written two or more kernels back): it copies
    // them and streams its first weights under g1's tail, the roles that touch what g1 wrote wait below
    if (!a.g2) griddep_wait();
    for (int i = tid; i < (int)(sizeof(RouteTables) / 4); i += kDThreads) ((int*)rt)[i] = ((const int*)a.rt)[i];
    __syncthreads();
    const int NB = a.NB, KS = a.K * 2 / 256;
    const uint32_t T = (uint32_t)(rt->n_active * NB * KS), G = T < gridDim.x ? T : gridDim.x;
    const bool part_of = blockIdx.x < G;
    const uint32_t lo = part_of ? blockIdx.x * T / G : 0u, hi = part_of ? (blockIdx.x + 1) * T / G : 0u;

    if (warp == 0) {
        if (lane == 0) {
            const uint64_t policy = policy_evict_first();
            uint32_t it = 0;
            for (uint32_t p = lo; p < hi && !*c.abort;) {
                const Item w = item_at(p, hi, T, G, (uint32_t)KS);
                p += (uint32_t)(w.k1 - w.k0);
                const int e = rt->act_e[w.u / NB], blk = w.u % NB;
                const unsigned char* src = a.w + ((size_t)(e * NB + blk) * KS + w.k0) * kStageW;
                for (int ks = w.k0; ks < w.k1; ++ks, ++it, src += kStageW) {
                    const uint32_t s = it % kBRing, round = it / kBRing;
                    if (!mbar_wait(&c.empty[s], (round & 1) ^ 1, c.abort)) {
                        dense_abort(c.status, c.abort, 600 + a.g2, (int)it);
                        break;
                    }
                    mbar_arrive_expect_tx(&c.full_w[s], 2 * kAtomW);
                    unsigned char* dst = c.wring + s * kStageW;
                    bulk_g2s_hint(dst, src, kAtomW, &c.full_w[s], policy);
                    bulk_g2s_hint(dst + kAtomW, src + kAtomW, kAtomW, &c.full_w[s], policy);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it = 0;
            int i = 0;
            for (uint32_t p = lo; p < hi && !*c.abort; ++i) {
                const Item w = item_at(p, hi, T, G, (uint32_t)KS);
                p += (uint32_t)(w.k1 - w.k0);
                const int buf = i & 1;
                if (!mbar_wait(&c.acc_empty[buf], ((i >> 1) & 1) ^ 1, c.abort)) {
                    dense_abort(c.status, c.abort, 610 + a.g2, i);
                    break;
                }
                tc_fence_after();
                const uint32_t d = c.tmem + buf * 16;
                bool ok = true;
                for (int ks = w.k0; ks < w.k1; ++ks, ++it) {
                    const uint32_t s = it % kBRing, round = it / kBRing;
                    if (!mbar_wait(&c.full_w[s], round & 1, c.abort) || !mbar_wait(&c.full_x[s], round & 1, c.abort)) {
                        dense_abort(c.status, c.abort, 620 + a.g2, (int)it);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t wb = smem_u32(c.wring + s * kStageW), xb = smem_u32(c.xring + s * kStageX);
#pragma unroll
                    for (int at = 0; at < 2; ++at)
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            mma_bf16(d, desc_sw128(wb + at * kAtomW + kk * 32), desc_sw128(xb + at * kAtomX + kk * 32),
                                     (ks != w.k0 || at != 0 || kk != 0) ? 1u : 0u);
                    tc_commit(&c.empty[s]);
                }
                if (!ok) break;
                tc_commit(&c.acc_full[buf]);
            }
        }
    } else if (warp < 4) {
        // ---- stager: the unit's rows of every stage, gathered by slot, kXDepth stages in flight per thread ----
        const int ts = tid - 64;
        if (a.g2) {
            griddep_wait();
            xchg_wait_role(a.wait, ts, 64, 3);  // every rank's column band of the h rows
        }
        uint32_t it = 0, arrived = 0;
        bool ok = true;
        for (uint32_t p = lo; p < hi && ok;) {
            const Item w = item_at(p, hi, T, G, (uint32_t)KS);
            p += (uint32_t)(w.k1 - w.k0);
            const int ai = w.u / NB, s0 = rt->act_off[ai], n_tok = rt->act_off[ai + 1] - s0;
            // this thread's four 16-byte chunks of a stage: row m = idx / 16 of the unit, the same for every stage
            const unsigned char* rows[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int m = (k * 64 + ts) >> 4;
                const int slot = m < n_tok ? rt->slot[s0 + m] : 0;
                rows[k] = (const unsigned char*)a.x + (size_t)(a.by_token ? slot / a.topk : slot) * a.K * 2;
            }
            for (int ks = w.k0; ks < w.k1; ++ks, ++it) {
                const uint32_t s = it % kBRing, round = it / kBRing;
                ok = mbar_wait(&c.empty[s], (round & 1) ^ 1, c.abort);
                if (!ok) {
                    dense_abort(c.status, c.abort, 630 + a.g2, (int)it);
                    break;
                }
                unsigned char* dst = c.xring + s * kStageX;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int idx = k * 64 + ts, m = idx >> 4, at = (idx >> 3) & 1, j = idx & 7;
                    // only live rows are written: a stale row feeds accumulator columns that no finish reads
                    if (m < n_tok)
                        cp_async16(dst + at * kAtomX + (m >> 3) * 1024 + (m & 7) * 128 + ((j ^ (m & 7)) << 4),
                                   rows[k] + (size_t)ks * 256 + at * 128 + j * 16, true);
                }
                cp_async_commit();
                if (it + 1 - arrived >= (uint32_t)kXDepth) {  // the stage issued kXDepth - 1 iterations ago has landed
                    cp_async_wait<kXDepth - 1>();
                    fence_proxy_async_smem();
                    mbar_arrive(&c.full_x[arrived % kBRing]);
                    ++arrived;
                }
            }
        }
        cp_async_wait<0>();
        fence_proxy_async_smem();
        if (ok)
            for (; arrived < it; ++arrived) mbar_arrive(&c.full_x[arrived % kBRing]);
    } else {
        // ---- epilogue ----
        if (a.g2) griddep_wait();
        const int q = warp - 4, te = tid - 128;
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        float* tile = c.tile;
        int i = 0;
        bool done = !(lo < hi);
        for (uint32_t p = lo; p < hi; ++i) {
            const Item w = item_at(p, hi, T, G, (uint32_t)KS);
            p += (uint32_t)(w.k1 - w.k0);
            const int buf = i & 1;
            if (!bar_all(2, 128, mbar_wait(&c.acc_full[buf], (i >> 1) & 1, c.abort))) {
                if (te == 0) dense_abort(c.status, c.abort, 640 + a.g2, i);
                break;
            }
            tc_fence_after();
            uint32_t r[16];
            tmem_ld16(c.tmem + lane_base + buf * 16, r);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(&c.acc_empty[buf]);
            float v[16];
#pragma unroll
            for (int m = 0; m < 16; ++m) v[m] = __uint_as_float(r[m]);
            bool finish = true;
            if (w.n > 1) {
                float* mine = a.part + piece_slot((int)blockIdx.x, w.c0) * 2048 + te;
#pragma unroll
                for (int m = 0; m < 16; ++m) __stcg(mine + m * 128, v[m]);
                __threadfence();
                bar_sync(2, 128);
                if (te == 0) *c.is_last = atomicInc(a.ticket + w.c0, (unsigned)(w.n - 1)) == (unsigned)(w.n - 1);
                bar_sync(2, 128);
                finish = *c.is_last != 0;
                if (finish) {
                    __threadfence();
#pragma unroll
                    for (int m = 0; m < 16; ++m) v[m] = 0.f;
                    for (int cc = w.c0; cc < w.c0 + w.n; ++cc) {
                        const float* src = a.part + piece_slot(cc, w.c0) * 2048 + te;
                        float t[16];
#pragma unroll
                        for (int m = 0; m < 16; ++m) t[m] = __ldcg(src + m * 128);
#pragma unroll
                        for (int m = 0; m < 16; ++m) v[m] += t[m];
                    }
                }
            }
            if (finish) {
#pragma unroll
                for (int m = 0; m < 16; ++m) tile[m * kTileLd + te] = v[m];
                bar_sync(2, 128);
                const int ai = w.u / NB, blk = w.u % NB, s0 = rt->act_off[ai], n_tok = rt->act_off[ai + 1] - s0;
                if (!a.g2) {
                    for (int idx = te; idx < 16 * 64; idx += 128) {
                        const int m = idx >> 6, j = idx & 63;
                        if (m >= n_tok) continue;
                        const float gv = bf16_round(tile[m * kTileLd + j]), uv = bf16_round(tile[m * kTileLd + 64 + j]);
                        const bf16 out = __float2bfloat16_rn((gv / (1.0f + expf(-gv))) * uv);
                        const size_t off = (size_t)rt->slot[s0 + m] * a.ldo + a.col0 + blk * 64 + j;
                        for (int d = 0; d < a.n_out; ++d) a.out[d][off] = out;
                    }
                } else {
                    for (int idx = te; idx < 16 * 128; idx += 128) {
                        const int m = idx >> 7, col = idx & 127;
                        if (m >= n_tok) continue;
                        const bf16 out = __float2bfloat16_rn(tile[m * kTileLd + col]);
                        const size_t off = (size_t)rt->slot[s0 + m] * a.ldo + a.col0 + blk * 128 + col;
                        for (int d = 0; d < a.n_out; ++d) a.out[d][off] = out;
                    }
                }
            }
            bar_sync(2, 128);  // the tile and the ticket flag are free again
            done = p >= hi;
        }
        if (te == 0 && !done && *c.abort == 0) dense_abort(c.status, c.abort, 650 + a.g2, i);
    }
    dense_teardown_cta(c);
    xchg_signal(a.sig);  // every CTA arrives, also one that had no unit
}

size_t experts_bf16_umma_smem() { return DenseLayout<kBRing>::kBytes + sizeof(RouteTables) + 16; }

cudaError_t experts_bf16_umma_prepare() {
    return cudaFuncSetAttribute(experts_bf16_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)experts_bf16_umma_smem());
}

cudaError_t experts_bf16_umma_launch(const Bf16UmmaArgs& a, int grid, cudaStream_t s, bool pdl) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kDThreads);
    cfg.dynamicSmemBytes = experts_bf16_umma_smem();
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, experts_bf16_umma_kernel, a);
}

}  // namespace mk
