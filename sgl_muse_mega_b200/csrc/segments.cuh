// Persistent "segment" kernels: the dense GEMMs of a layer and the row work between them in two launches instead of ten.
//
// The layer's dense GEMMs (o_proj, pooler, router, unpooler, qkv: 96 MB of weights at M <= 16 rows) are each far too short
// to amortise a launch, a cluster placement and a tail of their own, and the row kernels between them (norms, routing,
// combine) are pure latency. A segment is ONE kernel of one 512-thread CTA per SM that walks a fixed list of stages with
// a grid barrier between dependent ones:
//
//   segment A (after attention)   o_proj -> all-reduce exchange -> post norm -> pooler + router -> pooler exchange ->
//                                 top-k + route tables + pre-expert norm / quantisation
//   segment B (after the experts) combine -> unpooler -> unpooler exchange -> cross-layer norm -> qkv -> qk norm, RoPE,
//                                 K/V append
//
// GEMM stages are cut into items of 64 weight rows x 512 k (16 rows x 512 k for the f32 router): a CTA streams its items
// through two shared-memory buffers with bulk copies (mbarrier completion), multiplies with mma.sync (weights as the
// 16-row operand, the window rows as the 8-column operand, as gemm.cu) and leaves f32 partial sums per K chunk in global
// scratch; the stage that follows sums the chunks in chunk order (a fixed order: results do not depend on timing) and
// applies the epilogue (bf16 rounding and peer stores, routing, norms, row ops). Weight tiles never depend on the
// predecessor, so the first items of a GEMM stage are requested BEFORE the grid barrier (and before the programmatic
// launch wait) that guards the activations.
//
// Every wait is bounded: the grid barrier and the copy barriers give up after a poll budget, record the site in the
// launch's status block and carry on (the outputs are then meaningless, nothing hangs).
//
// This file is compiled as part of rows.cu: the segments reuse its row functions (top-k, route tables, quantisation).
#pragma once

#include "draft_rows.cuh"
#include "umma.cuh"

namespace mk {

constexpr int kSegThreads = 512;
constexpr int kSegWarps = kSegThreads / 32;
constexpr int kChunkK = 512;                          // k per GEMM item
constexpr int kSegPieces = 8;                         // bulk copies per packed item image (69,632 or 33,792 bytes)
constexpr int kSegBufBytes = 80 * (kChunkK * 2 + 64); // 64 weight + 16 activation rows of bf16 (f32: 16 + 16 rows fit too)
constexpr int kSegRedFloats = kSegWarps * 8 * 32;     // per-warp accumulator exchange
constexpr size_t kSegSmem = 2 * (size_t)kSegBufBytes + kSegRedFloats * 4 + 1024;

__host__ __device__ inline int seg_bn(const SegGemm& g) { return g.f32 ? 16 : 64; }
__host__ __device__ inline int seg_items(const SegGemm& g) { return ((g.N + seg_bn(g) - 1) / seg_bn(g)) * (g.K / kChunkK); }

// All threads of all CTAs. `site` is recorded when the wait runs out (status code 2).
__device__ __forceinline__ void grid_barrier(const GridBarrier& gb, int site) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned long long n = gridDim.x;
        const unsigned long long old = atomicAdd(gb.count, 1ull);
        const unsigned long long target = (old / n + 1) * n;
        long long polls = 0;
        while (*(volatile unsigned long long*)gb.count < target) {
            if (++polls > gb.budget) {
                if (gb.status != nullptr && atomicCAS(gb.status, 0, 2) == 0) {
                    gb.status[1] = site;
                    gb.status[2] = (int)blockIdx.x;
                }
                break;
            }
        }
        __threadfence();
    }
    __syncthreads();
}

// The CTA's streaming state: two buffers, their copy barriers and phases.
struct SegPipe {
    unsigned char* buf[2];
    float* red;
    uint64_t* bar;  // [2]; a phase completes with the weight request's arrival and bytes and one arrival per thread for its
                    // share of the activation rows
    int* abort;
    uint32_t phase[2];
    int* status;
    int tn;  // item-trace cursor (SEG_TRACE_ITEMS builds only)
};

__device__ __forceinline__ int seg_row_bytes(const SegGemm& g) { return kChunkK * (g.f32 ? 4 : 2) + 64; }

// Requests item `item`'s weight rows into buffer b (no dependency on any predecessor).
__device__ __forceinline__ void seg_issue_w(const SegGemm& g, int item, SegPipe& p, int b) {
    const int nsplit = g.K / kChunkK, nb = item / nsplit, ks = item - nb * nsplit;
    const int bn = seg_bn(g), es = g.f32 ? 4 : 2, rowb = seg_row_bytes(g);
    const int valid = min(bn, g.N - nb * bn);
    const int tid = threadIdx.x;
    if (g.packed) {  // the item's image is contiguous, padded rows included: a few large copies instead of one per row
        const uint32_t img = (uint32_t)(bn * rowb), piece = img / kSegPieces;
        if (tid == 0) umma::mbar_arrive_expect_tx(&p.bar[b], img);
        if (tid < kSegPieces) umma::bulk_g2s(p.buf[b] + tid * piece, g.w + (size_t)item * img + tid * piece, piece, &p.bar[b]);
        return;
    }
    if (tid < valid)
        umma::bulk_g2s(p.buf[b] + tid * rowb, g.w + (size_t)(nb * bn + tid) * g.ldw + (size_t)ks * kChunkK * es, kChunkK * es,
                       &p.bar[b]);
    if (tid == 0) umma::mbar_arrive_expect_tx(&p.bar[b], (uint32_t)(valid * kChunkK * es));
}

// Requests item `item`'s activation slice (M rows x one K chunk, at most 16 KB of bf16) into buffer b: every thread copies
// 32 bytes (64 for the f32 router) with cp.async and hands their completion to the buffer's barrier, which therefore
// counts one arrival per thread besides the weight request. (Sixteen small bulk copies per item kept the copy engine
// busier than the item's weights did.) Rows past the window and weight rows past N keep whatever the buffer held: an MMA
// output depends on its own weight row and its own window row only, and outputs outside [0, M) x [0, N) are never stored.
__device__ __forceinline__ void seg_issue_x(const SegGemm& g, int item, SegPipe& p, int b) {
    const int nsplit = g.K / kChunkK, ks = item % nsplit;
    const int bn = seg_bn(g), es = g.f32 ? 4 : 2, rowb = seg_row_bytes(g), per_row = kChunkK * es / 16;
    const int n = g.f32 ? 4 : 2;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (j >= n) break;
        const int piece = threadIdx.x + j * kSegThreads, m = piece / per_row, c = piece - m * per_row;
        if (m < g.M) cp_async16(p.buf[b] + (bn + m) * rowb + c * 16, g.x + (size_t)m * g.ldx + (size_t)ks * kChunkK * es + c * 16, true);
    }
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(umma::smem_u32(&p.bar[b])) : "memory");
}

// Multiplies the item in buffer b and stores its partial sums. All threads.
template <bool WF32>
__device__ __forceinline__ void seg_compute(const SegGemm& g, int item, SegPipe& p, int b) {
    constexpr int WN = WF32 ? 1 : 4, WK = kSegWarps / WN, ES = WF32 ? 4 : 2, KSTEP = 64 / ES, BN = 16 * WN;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, t = lane & 3;
    const int wn = warp % WN, wk = warp / WN;
    const int nsplit = g.K / kChunkK, nb = item / nsplit, ks = item - nb * nsplit;
    const int rowb = kChunkK * ES + 64;
    if (!umma::mbar_wait(&p.bar[b], p.phase[b], p.abort)) {
        if (atomicExch(p.abort, 1) == 0 && p.status != nullptr && atomicCAS(p.status, 0, 3) == 0) {
            p.status[1] = 210;
            p.status[2] = (int)blockIdx.x;
            p.status[3] = item;
        }
    }
    p.phase[b] ^= 1u;
#ifdef SEG_TRACE_ITEMS
    if (blockIdx.x == 0 && threadIdx.x == 0 && p.status && p.tn < 62) { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); ((unsigned long long*)(p.status + 64))[32 + p.tn++] = t; }
#endif
    constexpr int kw = kChunkK / WK, nsteps = kw / KSTEP;
    const unsigned char* wa0 = p.buf[b] + (wn * 16 + gq) * rowb + (wk * kw) * ES + t * 16;
    const unsigned char* wa1 = wa0 + 8 * rowb;
    const unsigned char* xs0 = p.buf[b] + (BN + gq) * rowb + (wk * kw) * ES + t * 16;
    const unsigned char* xs1 = xs0 + 8 * rowb;
    float acc0[4] = {0, 0, 0, 0}, acc1[4] = {0, 0, 0, 0};
    const bool two = g.M > 8;
#pragma unroll
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
    // the K warps of a row group meet in shared memory, in warp order
    {
        float* r = p.red + ((wk * WN + wn) * 8) * 32 + lane;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            r[i * 32] = acc0[i];
            r[(4 + i) * 32] = acc1[i];
        }
    }
    __syncthreads();
    // accumulator register i of lane ln of row group rn holds (row ln/4 + 8 (i/2 % 2), window row 8 (i/4) + 2 (ln%4) + i%2)
    float* part = g.part + (size_t)ks * 16 * g.N;
    for (int e = tid; e < WN * 256; e += kSegThreads) {
        const int rn = e >> 8, i = (e >> 5) & 7, ln = e & 31;
        float v = 0.f;
#pragma unroll
        for (int k = 0; k < WK; ++k) v += p.red[((k * WN + rn) * 8 + i) * 32 + ln];
        const int n = nb * BN + rn * 16 + (ln >> 2) + 8 * ((i >> 1) & 1);
        const int m = (i >> 2) * 8 + 2 * (ln & 3) + (i & 1);
        if (m < g.M && n < g.N) part[(size_t)m * g.N + n] = v;
    }
    __syncthreads();  // the buffer and the exchange area are free again
#ifdef SEG_TRACE_ITEMS
    if (blockIdx.x == 0 && threadIdx.x == 0 && p.status && p.tn < 62) { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); ((unsigned long long*)(p.status + 64))[32 + p.tn++] = t; }
#endif
}

// One GEMM stage: this CTA's items (cta, cta + grid, ...). `w_issued` items (0, 1 or 2) already have their weights on the
// way (seg_prefetch_w before the barrier that guards the activations).
__device__ __forceinline__ void seg_prefetch_w(const SegGemm& g, SegPipe& p, int first_item, int stride, int total) {
    if (first_item < total) seg_issue_w(g, first_item, p, 0);
    if (first_item + stride < total) seg_issue_w(g, first_item + stride, p, 1);
}

__device__ __forceinline__ void seg_gemm_stage(const SegGemm& g, SegPipe& p, int first_item, int stride, int total, bool w_issued) {
    int it0 = first_item, it1 = first_item + stride;
    if (it0 < total) {
        if (!w_issued) seg_issue_w(g, it0, p, 0);
        seg_issue_x(g, it0, p, 0);
    }
    if (it1 < total) {
        if (!w_issued) seg_issue_w(g, it1, p, 1);
        seg_issue_x(g, it1, p, 1);
    }
    int b = 0;
    for (int it = first_item; it < total; it += stride, b ^= 1) {
        if (g.f32) seg_compute<true>(g, it, p, b);
        else seg_compute<false>(g, it, p, b);
        const int nxt = it + 2 * stride;
        if (nxt < total) {
            seg_issue_w(g, nxt, p, b);
            seg_issue_x(g, nxt, p, b);
        }
    }
}

// A stage made of up to two GEMMs: items [0, n0) belong to g[0], the rest to g[1].
struct SegStage {
    SegGemm g[2];
    int n0, total;
};
__device__ __forceinline__ void seg_stage_issue_w(const SegStage& s, int item, SegPipe& p, int b) {
    if (item < s.n0) seg_issue_w(s.g[0], item, p, b);
    else seg_issue_w(s.g[1], item - s.n0, p, b);
}
__device__ __forceinline__ void seg_stage_issue_x(const SegStage& s, int item, SegPipe& p, int b) {
    if (item < s.n0) seg_issue_x(s.g[0], item, p, b);
    else seg_issue_x(s.g[1], item - s.n0, p, b);
}
__device__ __forceinline__ void seg_stage_prefetch_w(const SegStage& s, SegPipe& p) {
    const int first = blockIdx.x, stride = gridDim.x;
    if (first < s.total) seg_stage_issue_w(s, first, p, 0);
    if (first + stride < s.total) seg_stage_issue_w(s, first + stride, p, 1);
}
// Runs the stage's items of this CTA; the weights of its first two items are already requested (seg_stage_prefetch_w).
__device__ __forceinline__ void seg_stage_run(const SegStage& s, SegPipe& p) {
    const int first = blockIdx.x, stride = gridDim.x;
    if (first < s.total) seg_stage_issue_x(s, first, p, 0);
    if (first + stride < s.total) seg_stage_issue_x(s, first + stride, p, 1);
    int b = 0;
    for (int it = first; it < s.total; it += stride, b ^= 1) {
        const bool second = it >= s.n0;
        const SegGemm& g = s.g[second ? 1 : 0];
        const int local = second ? it - s.n0 : it;
        if (g.f32) seg_compute<true>(g, local, p, b);
        else seg_compute<false>(g, local, p, b);
        const int nxt = it + 2 * stride;
        if (nxt < s.total) {
            seg_stage_issue_w(s, nxt, p, b);
            seg_stage_issue_x(s, nxt, p, b);
        }
    }
}

// ---- finishes: sum the K chunks in chunk order, then the epilogue -----------------------------------------------------------

// out[m, col0 + n] = bf16(sum_ks part[ks][m][n]) into every destination (own buffer and peers'); all CTAs share the work.
__device__ __forceinline__ void seg_finish_bf16(const SegGemm& g, bf16* const* out, int n_out, long long ldo, long long off0) {
    const int nsplit = g.K / kChunkK;
    const long long total = (long long)g.M * g.N;
    for (long long i = (long long)blockIdx.x * kSegThreads + threadIdx.x; i < total; i += (long long)gridDim.x * kSegThreads) {
        const int m = (int)(i / g.N), n = (int)(i - (long long)m * g.N);
        float v = 0.f;
        for (int ks = 0; ks < nsplit; ++ks) v += g.part[((size_t)ks * 16 + m) * g.N + n];
        const bf16 b = __float2bfloat16_rn(v);
        for (int d = 0; d < n_out; ++d) out[d][off0 + (long long)m * ldo + n] = b;
    }
}

// SwiGLU over a [gate rows | up rows] GEMM: out[m, n] = bf16(silu(bf16(gate[m, n])) x bf16(up[m, n])), n < N / 2; f32 steps
// in the order gate / (1 + exp(-gate)) x up.
__device__ __forceinline__ void seg_finish_silu(const SegGemm& g, bf16* const* out, int n_out, long long ldo, long long off0) {
    const int nsplit = g.K / kChunkK, half = g.N / 2;
    const long long total = (long long)g.M * half;
    for (long long i = (long long)blockIdx.x * kSegThreads + threadIdx.x; i < total; i += (long long)gridDim.x * kSegThreads) {
        const int m = (int)(i / half), n = (int)(i - (long long)m * half);
        float gate = 0.f, up = 0.f;
        for (int ks = 0; ks < nsplit; ++ks) {
            const float* row = g.part + ((size_t)ks * 16 + m) * g.N;
            gate += row[n];
            up += row[half + n];
        }
        gate = bf16_round(gate);
        up = bf16_round(up);
        const bf16 b = __float2bfloat16_rn(__fmul_rn(__fdiv_rn(gate, __fadd_rn(1.0f, expf(-gate))), up));
        for (int d = 0; d < n_out; ++d) out[d][off0 + (long long)m * ldo + n] = b;
    }
}

// out[m, off0 + n] = sum_ks part[ks][m][n] as f32 into every destination (the lm_head's gathered logits); all CTAs share the
// work.
__device__ __forceinline__ void seg_finish_f32_push(const SegGemm& g, bf16* const* out, int n_out, long long ldo, long long off0) {
    const int nsplit = g.K / kChunkK;
    const long long total = (long long)g.M * g.N;
    for (long long i = (long long)blockIdx.x * kSegThreads + threadIdx.x; i < total; i += (long long)gridDim.x * kSegThreads) {
        const int m = (int)(i / g.N), n = (int)(i - (long long)m * g.N);
        float v = 0.f;
        for (int ks = 0; ks < nsplit; ++ks) v += g.part[((size_t)ks * 16 + m) * g.N + n];
        for (int d = 0; d < n_out; ++d) ((float*)out[d])[off0 + (long long)m * ldo + n] = v;
    }
}

// A conv projection (N = 2 sides x 2 taps x groups coefficient columns): the bf16 coefficients into c_out, then the conv's
// side 0 over the rows the projection was computed from, a thread per (row, group):
//   xa[m, ch] = (base[0, ch] + c[m, side 0, tap 0, g]) h[m, ch] + (base[1, ch] + c[m, side 0, tap 1, g]) h[m - 1, ch]
// in f32 with separately rounded products, as the stand-alone conv kernel.
__device__ __forceinline__ void seg_finish_conv(const SegGemm& g, bf16* c_out, long long ldo, const SegConv& cv) {
    const int nsplit = g.K / kChunkK;
    const long long total = (long long)g.M * g.N;
    for (long long i = (long long)blockIdx.x * kSegThreads + threadIdx.x; i < total; i += (long long)gridDim.x * kSegThreads) {
        const int m = (int)(i / g.N), n = (int)(i - (long long)m * g.N);
        float v = 0.f;
        for (int ks = 0; ks < nsplit; ++ks) v += g.part[((size_t)ks * 16 + m) * g.N + n];
        c_out[(long long)m * ldo + n] = __float2bfloat16_rn(v);
    }
    const int per_group = cv.H / cv.groups, pairs = g.M * cv.groups;
    for (int i = blockIdx.x * kSegThreads + threadIdx.x; i < pairs; i += gridDim.x * kSegThreads) {
        const int m = i / cv.groups, gi = i - m * cv.groups;
        float d0 = 0.f, d1 = 0.f;
        for (int ks = 0; ks < nsplit; ++ks) {
            const float* row = g.part + ((size_t)ks * 16 + m) * g.N;
            d0 += row[gi];
            d1 += row[cv.groups + gi];
        }
        d0 = bf16_round(d0);
        d1 = bf16_round(d1);
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

// The draft's qkv: a warp per (row, 128-wide head) sums its partial sums, rounds them to bf16 (the stored qkv row), then
// head norm, neox RoPE and the K / V append (dqkv_head).
__device__ __forceinline__ void seg_finish_dqkv(const SegGemm& g, bf16* qkv_out, long long ldo, const DQkvRowsArgs& a) {
    const int nsplit = g.K / kChunkK, heads = a.qh + 2 * a.kvh, lane = threadIdx.x & 31;
    const long long P = a.words[kWordP];
    for (int w = blockIdx.x * kSegWarps + (threadIdx.x >> 5); w < g.M * heads; w += gridDim.x * kSegWarps) {
        const int m = w / heads, head = w - m * heads;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        for (int ks = 0; ks < nsplit; ++ks) {
            const float* row = g.part + ((size_t)ks * 16 + m) * g.N + head * kDraftHeadDim;
            const float2 lo = *(const float2*)(row + 2 * lane), hi = *(const float2*)(row + 64 + 2 * lane);
            v[0] += lo.x;
            v[1] += lo.y;
            v[2] += hi.x;
            v[3] += hi.y;
        }
        const __nv_bfloat162 ql = __floats2bfloat162_rn(v[0], v[1]), qh = __floats2bfloat162_rn(v[2], v[3]);
        bf16* orow = qkv_out + (long long)m * ldo + head * kDraftHeadDim;
        *(__nv_bfloat162*)(orow + 2 * lane) = ql;
        *(__nv_bfloat162*)(orow + 64 + 2 * lane) = qh;
        v[0] = __low2float(ql);
        v[1] = __high2float(ql);
        v[2] = __low2float(qh);
        v[3] = __high2float(qh);
        dqkv_head(a, m, head, v, P, lane);
    }
}

// logits[m, n] = sum_ks part[ks][m][n] (f32), by one CTA.
__device__ __forceinline__ void seg_finish_f32_cta(const SegGemm& g, float* out) {
    const int nsplit = g.K / kChunkK;
    for (int i = threadIdx.x; i < g.M * g.N; i += kSegThreads) {
        const int m = i / g.N, n = i - m * g.N;
        float v = 0.f;
        for (int ks = 0; ks < nsplit; ++ks) v += g.part[((size_t)ks * 16 + m) * g.N + n];
        out[(size_t)m * g.N + n] = v;
    }
}

// The qkv epilogue (as gemm.cu mode 1): one warp per (row, head); bf16(acc), per-head qk norm (q scaled), interleaved-pair
// RoPE, K and V rows appended to the successor's pool.
__device__ __forceinline__ void seg_finish_qkv(const SegGemm& g, const GemmArgs& e) {
    const int nsplit = g.K / kChunkK, heads = g.N / kHeadDim;
    const int lane = threadIdx.x & 31;
    for (int w = blockIdx.x * kSegWarps + (threadIdx.x >> 5); w < g.M * heads; w += gridDim.x * kSegWarps) {
        const int m = w / heads, head = w - m * heads;
        float y0 = 0.f, y1 = 0.f;
        for (int ks = 0; ks < nsplit; ++ks) {
            const float2 v = *(const float2*)(g.part + ((size_t)ks * 16 + m) * g.N + head * kHeadDim + 2 * lane);
            y0 += v.x;
            y1 += v.y;
        }
        y0 = bf16_round(y0);
        y1 = bf16_round(y1);
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

// ---- row stages for a 512-thread CTA -----------------------------------------------------------------------------------------

// resid_norm_kernel's arithmetic for one row: thread t owns columns (j 512 + t) 8 .. + 7 of chunk j (H <= 8192).
__device__ __forceinline__ void seg_norm_row(const NormArgs& a, int row, float* red) {
    const int tid = threadIdx.x;
    float v[2][8], ns[2][8];
    bool on[2];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int c0 = (j * kSegThreads + tid) * 8;
        on[j] = c0 < a.H;
        if (!on[j]) continue;
        const size_t off = (size_t)row * a.H + c0;
        if (a.mode == 0) {
            unpack8(*(const uint4*)(a.src + ((size_t)0 * a.M + row) * a.H + c0), v[j]);
            for (int r = 1; r < a.ranks; ++r) {
                float f[8];
                unpack8(*(const uint4*)(a.src + ((size_t)r * a.M + row) * a.H + c0), f);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[j][i] += f[i];
            }
            const uint4 b = pack8(v[j]);
            *(uint4*)(a.branch + off) = b;
            unpack8(b, v[j]);
        } else {
            float w[8];
            unpack8(*(const uint4*)(a.src + off), v[j]);
            unpack8(*(const uint4*)(a.post_w + c0), w);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[j][i] *= w[i];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += v[j][i] * v[j][i];
    }
    const float post_rstd = inv_sqrt(block_sum(ss, red) / (float)a.H + 1e-8f);
    ss = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        if (!on[j]) continue;
        const int c0 = (j * kSegThreads + tid) * 8;
        const size_t off = (size_t)row * a.H + c0;
        const float4 s0 = *(const float4*)(a.stream_in + off), s1 = *(const float4*)(a.stream_in + off + 4);
        const float4 al0 = *(const float4*)(a.alpha + c0), al1 = *(const float4*)(a.alpha + c0 + 4);
        const float4 be0 = *(const float4*)(a.beta + c0), be1 = *(const float4*)(a.beta + c0 + 4);
        const float st[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        const float al[8] = {al0.x, al0.y, al0.z, al0.w, al1.x, al1.y, al1.z, al1.w};
        const float be[8] = {be0.x, be0.y, be0.z, be0.w, be1.x, be1.y, be1.z, be1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float scaled = a.mode == 0 ? (be[i] * post_rstd) * v[j][i] : be[i] * (v[j][i] * post_rstd);
            ns[j][i] = fmaf(al[i], st[i], scaled);
            ss += ns[j][i] * ns[j][i];
        }
        *(float4*)(a.stream_out + off) = make_float4(ns[j][0], ns[j][1], ns[j][2], ns[j][3]);
        *(float4*)(a.stream_out + off + 4) = make_float4(ns[j][4], ns[j][5], ns[j][6], ns[j][7]);
    }
    const float pre_rstd = inv_sqrt(block_sum(ss, red) / (float)a.H + 1e-5f);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        if (!on[j]) continue;
        const int c0 = (j * kSegThreads + tid) * 8;
        const size_t off = (size_t)row * a.H + c0;
        float pw[8], h[8];
        unpack8(*(const uint4*)(a.pre_w + c0), pw);
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = (ns[j][i] * pre_rstd) * pw[i];
        const uint4 hb = pack8(h);
        *(uint4*)(a.normed + off) = hb;
        if (a.normed_f32) {
            unpack8(hb, h);
            *(float4*)(a.normed_f32 + off) = make_float4(h[0], h[1], h[2], h[3]);
            *(float4*)(a.normed_f32 + off + 4) = make_float4(h[4], h[5], h[6], h[7]);
        }
    }
}

// combine_kernel's arithmetic for one row: thread t owns columns 8 t .. 8 t + 7 (P <= 4096).
__device__ __forceinline__ void seg_combine_row(const CombineArgs& a, int row, float (*redk)[kSegWarps + 1], float* sc) {
    const int tid = threadIdx.x, c0 = tid * 8, warp = tid >> 5, lane = tid & 31;
    const bool on = c0 < a.P;
    if (row >= a.b_live) {
        if (on) *(uint4*)(a.y + (size_t)row * a.P + c0) = make_uint4(0, 0, 0, 0);
        return;
    }
    float gp[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (on) unpack8(*(const uint4*)(a.gamma_p1 + c0), gp);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j0 = 0; j0 < a.k; j0 += kMaxTopk) {
        const int kk = min(kMaxTopk, a.k - j0);
        float xg[kMaxTopk][8];
#pragma unroll
        for (int j = 0; j < kMaxTopk; ++j) {
            float ss = 0.f;
            if (j < kk) {
                if (on) unpack8(*(const uint4*)(a.zb + ((size_t)row * a.k + j0 + j) * a.P + c0), xg[j]);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    xg[j][i] = on ? xg[j][i] * gp[i] : 0.f;
                    ss += xg[j][i] * xg[j][i];
                }
            }
            ss = warp_sum(ss);
            if (lane == 0) redk[j][warp] = ss;
        }
        __syncthreads();
        if (tid < kMaxTopk && tid < kk) {
            float s = 0.f;
            for (int w = 0; w < kSegWarps; ++w) s += redk[tid][w];
            sc[tid] = a.w[(size_t)row * a.k + j0 + tid] * (1.0f / sqrtf(s / (float)a.P + 1e-8f));
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < kMaxTopk; ++j)
            if (j < kk) {
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] = fmaf(sc[j], xg[j][i], acc[i]);
            }
        __syncthreads();
    }
    if (on) *(uint4*)(a.y + (size_t)row * a.P + c0) = pack8(acc);
}

// Stage timestamps of CTA 0 (nanoseconds of the global timer) in words [64, 128) of the launch's status block: segment A
// uses slots 0..15, segment B 16..31. Read by the profiling notes; costs one store per stage.
__device__ __forceinline__ void seg_trace(int* status, int slot) {
    if (status != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        ((unsigned long long*)(status + 64))[slot] = t;
    }
}

struct SegShared {
    uint64_t bar[2];
    int abort;
    float red[33];
    float redk[kMaxTopk][kSegWarps + 1];
    float sc[kMaxTopk];
    int s_ids[kMaxSlots];
    int cnt[1024];
    int first[1024];
};

__device__ __forceinline__ void seg_setup(SegPipe& p, SegShared& sh, unsigned char* dyn, int* status) {
    p.buf[0] = dyn;
    p.buf[1] = dyn + kSegBufBytes;
    p.red = (float*)(dyn + 2 * kSegBufBytes);
    p.bar = sh.bar;
    p.abort = &sh.abort;
    p.phase[0] = p.phase[1] = 0;
    p.status = status;
    p.tn = 0;
    if (threadIdx.x == 0) {
        sh.abort = 0;
        umma::mbar_init(&sh.bar[0], 1 + kSegThreads);
        umma::mbar_init(&sh.bar[1], 1 + kSegThreads);
        umma::mbar_fence_init();
    }
    __syncthreads();
}

// ---- one GEMM stage as a kernel of its own --------------------------------------------------------------------------------------
// The same item engine behind one grid barrier and a finish, for the per-stage launch list: o_proj (bf16 push into the
// all-reduce workspaces), pooler + router in one launch (bf16 push into the node's gather rows; f32 logits and the routing's
// selection scores), unpooler (bf16 push), qkv (row ops). The row kernels around them stay separate launches.
__global__ void __launch_bounds__(kSegThreads, 1) seg_gemm_kernel(const SegGemmArgs a) {
    extern __shared__ __align__(128) unsigned char dyn[];
    __shared__ SegShared sh;
    SegPipe p;
    seg_setup(p, sh, dyn, a.status);
    SegStage st{{a.g[0], a.g[a.n_gemm > 1 ? 1 : 0]}, seg_items(a.g[0]), seg_items(a.g[0]) + (a.n_gemm > 1 ? seg_items(a.g[1]) : 0)};
    seg_stage_prefetch_w(st, p);  // static weights: requested while the predecessor still runs
    griddep_wait();
    seg_stage_run(st, p);
    grid_barrier(a.gb, 30 + a.finish);
    if (a.finish == 2) {
        seg_finish_qkv(a.g[0], a.epi);
    } else if (a.finish == 3) {
        seg_finish_silu(a.g[0], a.out, a.n_out, a.ldo, a.off0);
    } else if (a.finish == 4) {
        seg_finish_f32_push(a.g[0], a.out, a.n_out, a.ldo, a.off0);
    } else if (a.finish == 5) {
        seg_finish_conv(a.g[0], a.out[0], a.ldo, a.conv);
    } else if (a.finish == 6) {
        seg_finish_dqkv(a.g[0], a.out[0], a.ldo, a.rows);
    } else {
        seg_finish_bf16(a.g[0], a.out, a.n_out, a.ldo, a.off0);
        if (a.finish == 1) {
            // the router: f32 logits and, a thread per logit, the routing's selection scores (sigmoid in f64 rounded to
            // f32, plus the expert's bias)
            const SegGemm& g = a.g[1];
            const int nsplit = g.K / kChunkK;
            for (int i = blockIdx.x * kSegThreads + threadIdx.x; i < g.M * g.N; i += gridDim.x * kSegThreads) {
                const int m = i / g.N, n = i - m * g.N;
                float v = 0.f;
                for (int ks = 0; ks < nsplit; ++ks) v += g.part[((size_t)ks * 16 + m) * g.N + n];
                a.f32_out[i] = v;
                if (a.score != nullptr) a.score[i] = (float)(1.0 / (1.0 + exp(-((double)v * a.score_mult)))) + a.score_bias[n];
            }
        }
    }
    xchg_signal(a.sig);
}

// ---- segment A -----------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kSegThreads, 1) segment_a_kernel(const SegAArgs a) {
    extern __shared__ __align__(128) unsigned char dyn[];
    __shared__ SegShared sh;
    SegPipe p;
    seg_setup(p, sh, dyn, a.status);
    const int cta = blockIdx.x;
    SegStage s1{{a.oproj, a.oproj}, seg_items(a.oproj), seg_items(a.oproj)};
    SegStage s3{{a.pooler, a.router}, seg_items(a.pooler), seg_items(a.pooler) + seg_items(a.router)};
    seg_trace(a.status, 0);
    seg_stage_prefetch_w(s1, p);  // static weights: on their way while the attention still runs
    griddep_wait();
    seg_trace(a.status, 1);
    // the exchanges this kernel both feeds and consumes: their epoch before any CTA of this launch can have signalled
    const unsigned e_ar = xchg_epoch(a.post_norm.wait) + 1, e_pool = xchg_epoch(a.nq.wait) + 1;
    seg_stage_run(s1, p);
    seg_trace(a.status, 2);
    seg_stage_prefetch_w(s3, p);
    grid_barrier(a.gb, 1);
    seg_trace(a.status, 3);
    // this rank's bf16 partial of the all-reduce, pushed into every present rank's workspace
    seg_finish_bf16(a.oproj, a.ar_out, a.n_ar, a.oproj.N, a.ar_off);
    xchg_signal(a.sig_ar);
    seg_trace(a.status, 4);
    if (cta < a.post_norm.M) {
        xchg_wait_epoch(a.post_norm.wait, e_ar);
        seg_norm_row(a.post_norm, cta, sh.red);
    }
    seg_trace(a.status, 5);
    grid_barrier(a.gb, 2);
    seg_trace(a.status, 6);
    seg_stage_run(s3, p);
    seg_trace(a.status, 7);
    grid_barrier(a.gb, 3);
    seg_trace(a.status, 8);
    seg_finish_bf16(a.pooler, a.pool_out, a.n_pool, a.pool_ld, a.pool_col0);
    xchg_signal(a.sig_pool);
    seg_trace(a.status, 9);
    if (cta == (int)gridDim.x - 1) {
        seg_finish_f32_cta(a.router, a.logits);
        __syncthreads();
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int row = warp; row < a.topk.M; row += kSegWarps) topk_row(a.topk, row, lane, sh.s_ids);
        __syncthreads();
        route_tables(sh.s_ids, a.topk.E, a.b_live * a.topk.k, a.rt, sh.cnt, sh.first, a.topk.e_lo, a.topk.e_hi);
    } else if (cta < a.topk.M) {
        xchg_wait_epoch(a.nq.wait, e_pool);
        nq_row(a.nq, cta, sh.red);
    }
    seg_trace(a.status, 10);
}

// ---- segment B -----------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kSegThreads, 1) segment_b_kernel(const SegBArgs a) {
    extern __shared__ __align__(128) unsigned char dyn[];
    __shared__ SegShared sh;
    SegPipe p;
    seg_setup(p, sh, dyn, a.status);
    const int cta = blockIdx.x;
    SegStage s2{{a.unpool, a.unpool}, seg_items(a.unpool), seg_items(a.unpool)};
    seg_trace(a.status, 16);
    seg_stage_prefetch_w(s2, p);
    griddep_wait();
    seg_trace(a.status, 17);
    const unsigned e_unpool = xchg_epoch(a.cross_norm.wait) + 1;  // fed and consumed by this kernel
    if (cta < a.M) {
        xchg_wait(a.combine.wait);
        seg_combine_row(a.combine, cta, sh.redk, sh.sc);
    }
    seg_trace(a.status, 18);
    grid_barrier(a.gb, 11);
    seg_trace(a.status, 19);
    seg_stage_run(s2, p);
    seg_trace(a.status, 20);
    SegStage s4{{a.qkv, a.qkv}, 0, 0};
    if (!a.tail) {
        s4.n0 = s4.total = seg_items(a.qkv);
        seg_stage_prefetch_w(s4, p);
    }
    grid_barrier(a.gb, 12);
    seg_trace(a.status, 21);
    seg_finish_bf16(a.unpool, a.unpool_out, a.n_unpool, a.unpool_ld, a.unpool_col0);
    xchg_signal(a.sig_unpool);
    if (cta < a.M) {
        xchg_wait_epoch(a.cross_norm.wait, e_unpool);
        seg_norm_row(a.cross_norm, cta, sh.red);
    }
    seg_trace(a.status, 22);
    if (a.tail) return;
    grid_barrier(a.gb, 13);
    seg_trace(a.status, 23);
    seg_stage_run(s4, p);
    seg_trace(a.status, 24);
    grid_barrier(a.gb, 14);
    seg_trace(a.status, 25);
    seg_finish_qkv(a.qkv, a.qkv_epi);
    seg_trace(a.status, 26);
}

size_t segments_smem() { return kSegSmem; }

cudaError_t segments_prepare() {
    cudaError_t e = cudaFuncSetAttribute(segment_a_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSegSmem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(segment_b_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSegSmem);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(seg_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSegSmem);
}

template <typename Args>
static cudaError_t seg_launch(void (*kern)(const Args), const Args& a, int grid, cudaStream_t s, bool pdl) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kSegThreads);
    cfg.dynamicSmemBytes = kSegSmem;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, a);
}
cudaError_t seg_gemm_launch(const SegGemmArgs& a, int grid, cudaStream_t s, bool pdl) {
    if (a.g[0].packed == 2) return dense_launch(a, grid, s, pdl);  // tile images: the tcgen05 engine of dense.cu
    return seg_launch(seg_gemm_kernel, a, grid, s, pdl);
}
cudaError_t seg_a_launch(const SegAArgs& a, int grid, cudaStream_t s, bool pdl) { return seg_launch(segment_a_kernel, a, grid, s, pdl); }
cudaError_t seg_b_launch(const SegBArgs& a, int grid, cudaStream_t s, bool pdl) { return seg_launch(segment_b_kernel, a, grid, s, pdl); }

}  // namespace mk
