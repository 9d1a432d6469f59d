// Two kernels per layer for everything that is not attention or experts: the dense GEMMs on the tensor-core engine of
// dense.cuh chained with the row work between them, one persistent CTA per SM.
//
//   kernel A (after attention)    o_proj -> all-reduce exchange -> post-attention norm rows -> pooler + router ->
//                                 pooler exchange -> top-k + route tables | pre-expert norm + quantisation rows
//   kernel B (after the experts)  combine rows -> unpooler -> unpooler exchange -> cross-layer norm rows -> qkv head
//                                 (qk norm, RoPE, K / V append in its epilogue)
//
// Both are the same program: [row stage] GEMM stage [row stage] GEMM stage [row stage]. The four roles of the engine walk
// the program independently: the weight producer and the MMA issuer run ahead into the next GEMM stage (its weights stream
// into the ring while the rows between the stages are still being computed: weights depend on nothing), the activation
// stager waits for the rows the next stage multiplies, the epilogue warps finish tiles and then work on the rows.
// Reference counterparts: sm103/kernels/layer.cu:213-237 (phase program), kernels/postattn.cuh:307-354 (unit queue),
// kernels/framework.cuh:1650-1692 (ticketed counts instead of grid barriers).
//
// Synchronisation is by counters that only grow (no grid barrier, no reset between launches):
//   * each kernel keeps, in the layer's private scratch, a launch count (bumped by the last CTA out) and dependency words;
//     a CTA reads the launch count e once at its start and waits for word >= (e + 1) x arrivals-per-launch;
//   * the exchanges a kernel both feeds and consumes (all-reduce, pooler gather, unpooler gather) get one arrival per
//     FINISHED TILE on every receiving rank, in words of the flag block that the per-stage kernels do not use; the
//     consumer rows wait for (e' + 1) x present ranks x tiles, e' the flag block's own launch count of that exchange.
// Every wait is bounded (poll budget), records itself in the status block (code 1 exchange, code 2 dependency word) and
// carries on; nothing traps.
//
// Row stages run on the 128 threads of the epilogue warps: a norm or combine row is cut into parts of 1024 columns, one part
// per CTA (the row's sums meet through the layer's scratch, in part order); a pre-expert row on CTA r, the routing on the
// last CTA. Their arithmetic is that of the row kernels of rows.cu (same rounding points; f32 sums in another fixed order).
//
// This file is compiled as part of rows.cu: the row stages reuse its top-k, route tables and number formats.
#pragma once

#include "dense.cuh"

namespace mk {

constexpr int kFRing = 5;  // weight / activation stages in flight (one less than the one-stage kernel: the row stages' scratch)

struct FusedShared {  // behind the engine's shared memory
    float red[33];
    float redk[kMaxTopk][5];
    float total[kMaxTopk];
    int s_ids[kMaxSlots];
    int cnt[1024];   // route tables; the top-k CTAs keep their row's selection scores here (as floats)
    int first[1024]; // route tables; the top-k CTAs keep the experts' biases here (as floats)
};

// ---- bounded waits on words that only grow -------------------------------------------------------------------------------------
// One thread of the group polls, the group meets at its barrier. `sys`: the word is written by other GPUs.
__device__ __forceinline__ void grp_wait_word(const unsigned* word, unsigned target, bool sys, long long budget, int* status, int code,
                                              int site, const Grp& g) {
    if (g.tid == 0) {
        long long polls = 0;
        for (;;) {
            unsigned seen;
            if (sys) asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(word) : "memory");
            else asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(word) : "memory");
            if ((int)(seen - target) >= 0) break;
            if ((polls & 1023) == 1023 && status != nullptr && *(volatile int*)status != 0) break;  // a failure is on record
            if (++polls > budget) {
                if (status != nullptr && atomicCAS(status, 0, code) == 0) {
                    status[1] = site;
                    status[2] = (int)blockIdx.x;
                    status[3] = (int)seen;
                    status[4] = (int)target;
                }
                break;
            }
            __nanosleep(32);
        }
    }
    grp_sync(g);
}

// the whole-kernel exchange wait of params.h for a thread group (the expert outputs the combine rows read)
__device__ __forceinline__ void grp_xchg_wait(const XchgWait& w, const Grp& g) {
    if (w.flag == nullptr) return;
    const unsigned epoch = *(volatile const unsigned*)w.epoch;
    grp_wait_word(w.flag, epoch * w.contributors, true, w.budget, w.status, 1, w.stage, g);
}

// after a group's global stores: make them visible, then one arrival on a dependency word of this GPU
__device__ __forceinline__ void grp_arrive(unsigned* word, const Grp& g) {
    __threadfence();
    grp_sync(g);
    if (g.tid == 0) atomicAdd(word, 1u);
}

// ---- row stages on a 128-thread group ----------------------------------------------------------------------------------------
// A row is cut into parts of 1024 columns, one part per CTA (a thread owns 8 consecutive columns, as in the row kernels
// of rows.cu, so nothing is kept in arrays). The sums over a whole row meet through the layer's scratch: every part
// stores its partial sum, arrives on the row's counter, waits for the row's other parts and adds the partial sums in part
// order (a fixed order: results do not depend on timing).
struct RowMeet {
    float* part;        // [rows][parts][width] partial sums
    unsigned* count;    // [rows] arrivals, only grows
    unsigned launch;    // this kernel's launch count at its start
    int parts, width;
    long long budget;
    int* status;
};
// `mine[0..width)` (thread 0 of the group holds them) -> `total[0..width)` in shared memory, for every thread of the group.
__device__ __forceinline__ void row_meet(const RowMeet& m, int row, int part, const float* mine, float* total, int site, const Grp& g) {
    if (m.parts == 1) {
        if (g.tid == 0)
            for (int i = 0; i < m.width; ++i) total[i] = mine[i];
        grp_sync(g);
        return;
    }
    if (g.tid == 0) {
        for (int i = 0; i < m.width; ++i) __stcg(m.part + ((size_t)row * m.parts + part) * m.width + i, mine[i]);
        __threadfence();
        atomicAdd(m.count + row, 1u);
    }
    grp_wait_word(m.count + row, (m.launch + 1) * (unsigned)m.parts, false, m.budget, m.status, 2, site, g);
    if (g.tid < m.width) {
        float s = 0.f;
        for (int p = 0; p < m.parts; ++p) s += __ldcg(m.part + ((size_t)row * m.parts + p) * m.width + g.tid);
        total[g.tid] = s;
    }
    grp_sync(g);
}

// resid_norm_kernel's arithmetic (rows.cu) for columns [1024 part, 1024 part + 1024) of one row, with ONE meeting of the
// row's parts: besides sum v^2 every part sums p^2, p q and q^2 of p = alpha x stream, q = beta x v, so that the second
// norm's sum of squares of ns = p + rstd q follows from the first norm's rstd without a second meeting:
// sum ns^2 = sum p^2 + 2 rstd sum p q + rstd^2 sum q^2 (equal to summing the rounded ns^2 up to f32 rounding of the sums).
__device__ __forceinline__ void norm_part_g(const NormArgs& a, int row, int part, const RowMeet& m1, float* red, float* total,
                                            const Grp& g) {
    const int c0 = (part * 128 + g.tid) * 8;
    const size_t off = (size_t)row * a.H + c0;
    // everything this part reads besides the rows it waited for: requested first
    const float4 s0 = *(const float4*)(a.stream_in + off), s1 = *(const float4*)(a.stream_in + off + 4);
    const float4 al0 = *(const float4*)(a.alpha + c0), al1 = *(const float4*)(a.alpha + c0 + 4);
    const float4 be0 = *(const float4*)(a.beta + c0), be1 = *(const float4*)(a.beta + c0 + 4);
    const uint4 pw_raw = *(const uint4*)(a.pre_w + c0);
    float v[8];
    if (a.mode == 0) {
        uint4 raw[kMaxRanks];
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
            if (r < a.ranks) raw[r] = *(const uint4*)(a.src + ((size_t)r * a.M + row) * a.H + c0);
        unpack8(raw[0], v);
#pragma unroll
        for (int r = 1; r < kMaxRanks; ++r)
            if (r < a.ranks) {
                float f[8];
                unpack8(raw[r], f);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] += f[i];
            }
        const uint4 b = pack8(v);
        *(uint4*)(a.branch + off) = b;
        unpack8(b, v);
    } else {
        float w[8];
        unpack8(*(const uint4*)(a.src + off), v);
        unpack8(*(const uint4*)(a.post_w + c0), w);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] *= w[i];
    }
    const float st[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const float al[8] = {al0.x, al0.y, al0.z, al0.w, al1.x, al1.y, al1.z, al1.w};
    const float be[8] = {be0.x, be0.y, be0.z, be0.w, be1.x, be1.y, be1.z, be1.w};
    float sv = 0.f, spp = 0.f, spq = 0.f, sqq = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float p = al[i] * st[i], q = be[i] * v[i];
        sv += v[i] * v[i];
        spp += p * p;
        spq += p * q;
        sqq += q * q;
    }
    // four group sums through one pass over shared memory: lane 0 of every warp holds its warp's sums
    sv = warp_sum(sv);
    spp = warp_sum(spp);
    spq = warp_sum(spq);
    sqq = warp_sum(sqq);
    grp_sync(g);
    if ((g.tid & 31) == 0) {
        float* r = red + (g.tid >> 5) * 4;
        r[0] = sv; r[1] = spp; r[2] = spq; r[3] = sqq;
    }
    grp_sync(g);
    float mine[4];
    if (g.tid == 0)
        for (int i = 0; i < 4; ++i) mine[i] = (red[i] + red[4 + i]) + (red[8 + i] + red[12 + i]);
    row_meet(m1, row, part, mine, total, 640, g);
    const float post_rstd = inv_sqrt(total[0] / (float)a.H + 1e-8f);
    const float ss2 = total[1] + 2.0f * post_rstd * total[2] + (post_rstd * post_rstd) * total[3];
    const float pre_rstd = inv_sqrt(ss2 / (float)a.H + 1e-5f);
    float ns[8], pw[8], h[8];
    unpack8(pw_raw, pw);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float scaled = a.mode == 0 ? (be[i] * post_rstd) * v[i] : be[i] * (v[i] * post_rstd);
        ns[i] = fmaf(al[i], st[i], scaled);
        h[i] = (ns[i] * pre_rstd) * pw[i];
    }
    *(float4*)(a.stream_out + off) = make_float4(ns[0], ns[1], ns[2], ns[3]);
    *(float4*)(a.stream_out + off + 4) = make_float4(ns[4], ns[5], ns[6], ns[7]);
    const uint4 hb = pack8(h);
    *(uint4*)(a.normed + off) = hb;
    if (a.normed_f32) {
        unpack8(hb, h);
        *(float4*)(a.normed_f32 + off) = make_float4(h[0], h[1], h[2], h[3]);
        *(float4*)(a.normed_f32 + off + 4) = make_float4(h[4], h[5], h[6], h[7]);
    }
    grp_sync(g);  // red / total are free again
}

// nq_row's arithmetic (rows.cu) for one 16-element group held in registers (lo / hi: its two 8-element halves).
#define MK_NQ_NORM8(v, graw, gmax)                                   \
    {                                                                \
        float gm_[8];                                                \
        unpack8(graw, gm_);                                          \
        _Pragma("unroll") for (int i_ = 0; i_ < 8; ++i_) {           \
            v[i_] = bf16_round(bf16_round(v[i_] * rstd) * gm_[i_]);  \
            gmax = fmaxf(gmax, fabsf(v[i_]));                        \
        }                                                            \
    }
#define MK_NQ_QUANT(lo_, hi_, gmax, gi)                                                              \
    {                                                                                                \
        const uint32_t sfb_ = float_to_e4m3((fmaxf(gmax, 1e-10f) * kSixth) * inv_x);                 \
        const float os_ = 1.0f / fmaxf(e4m3_to_float(sfb_) * x_scale, 1e-10f);                       \
        uint32_t l_ = 0, h_ = 0;                                                                     \
        _Pragma("unroll") for (int i_ = 0; i_ < 8; ++i_) {                                           \
            l_ |= float_to_e2m1(lo_[i_] * os_) << (4 * i_);                                          \
            h_ |= float_to_e2m1(hi_[i_] * os_) << (4 * i_);                                          \
        }                                                                                            \
        *(uint2*)(a.q + (size_t)row * (a.P / 2) + (gi) * 8) = make_uint2(l_, h_);                    \
        a.sf[(size_t)row * groups + (gi)] = (unsigned char)sfb_;                                     \
    }
#ifdef FUSED_TRACE
#define NQ_T(slot)                                                                   \
    if (g.tid == 0 && blockIdx.x == 0 && trace != nullptr) {                         \
        unsigned long long t_;                                                       \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                      \
        ((unsigned long long*)trace)[32 + (slot)] = t_;                              \
    }
#else
#define NQ_T(slot)
#endif
// Up to two groups per thread (P <= 4096): group t and group t + 128.
__device__ __forceinline__ void nq_row_g(const NqArgs& a, int row, float* red, const Grp& g, int* trace = nullptr) {
    const int t = g.tid, groups = a.P / 16;
    const bf16* x = a.pooled + (size_t)row * a.P;
    const bool on0 = t < groups, on1 = t + 128 < groups;
    float lo0[8], hi0[8], lo1[8], hi1[8];
    uint4 g0a = make_uint4(0, 0, 0, 0), g0b = g0a, g1a = g0a, g1b = g0a;  // the norm weights: requested with the row
    float ss = 0.f;
    if (on0) {
        unpack8(*(const uint4*)(x + t * 16), lo0);
        unpack8(*(const uint4*)(x + t * 16 + 8), hi0);
        g0a = *(const uint4*)(a.gamma + t * 16);
        g0b = *(const uint4*)(a.gamma + t * 16 + 8);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += lo0[i] * lo0[i];
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += hi0[i] * hi0[i];
    }
    if (on1) {
        unpack8(*(const uint4*)(x + (t + 128) * 16), lo1);
        unpack8(*(const uint4*)(x + (t + 128) * 16 + 8), hi1);
        g1a = *(const uint4*)(a.gamma + (t + 128) * 16);
        g1b = *(const uint4*)(a.gamma + (t + 128) * 16 + 8);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += lo1[i] * lo1[i];
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += hi1[i] * hi1[i];
    }
    NQ_T(12)
    const float rstd = inv_sqrt(grp_sum(ss, red, g) / (float)a.P + a.eps);
    NQ_T(13)
    float gmax0 = 0.f, gmax1 = 0.f;
    if (on0) {
        MK_NQ_NORM8(lo0, g0a, gmax0)
        MK_NQ_NORM8(hi0, g0b, gmax0)
    }
    if (on1) {
        MK_NQ_NORM8(lo1, g1a, gmax1)
        MK_NQ_NORM8(hi1, g1b, gmax1)
    }
    if (a.bf16_out) {
        if (on0) {
            bf16* o = (bf16*)a.q + (size_t)row * a.P + t * 16;
            *(uint4*)o = pack8(lo0);
            *(uint4*)(o + 8) = pack8(hi0);
        }
        if (on1) {
            bf16* o = (bf16*)a.q + (size_t)row * a.P + (t + 128) * 16;
            *(uint4*)o = pack8(lo1);
            *(uint4*)(o + 8) = pack8(hi1);
        }
        return;
    }
    NQ_T(16)
    const float amax = grp_max(fmaxf(gmax0, gmax1), red, g);
    NQ_T(17)
    const float kSixth = 1.0f / 6.0f, kInv2688 = 1.0f / 2688.0f;
    const float x_scale = fmaxf(amax, 1e-10f) * kInv2688;
    const float inv_x = 1.0f / x_scale;
    if (t == 0) a.x_scale[row] = x_scale;
    if (on0) MK_NQ_QUANT(lo0, hi0, gmax0, t)
    if (on1) MK_NQ_QUANT(lo1, hi1, gmax1, t + 128)
}

// combine_kernel's arithmetic (rows.cu) for columns [1024 part, 1024 part + 1024) of one row: the k slot rows' chunks stay in
// registers, the k sums of squares meet across the row's parts (k <= 8).
__device__ __forceinline__ void combine_part_g(const CombineArgs& a, int row, int part, const RowMeet& m, float (*redk)[5], float* total,
                                               const Grp& g) {
    const int t = g.tid, warp = t >> 5, lane = t & 31, c0 = (part * 128 + t) * 8;
    const bool on = c0 < a.P;
    if (row >= a.b_live) {
        if (on) *(uint4*)(a.y + (size_t)row * a.P + c0) = make_uint4(0, 0, 0, 0);
        return;
    }
    float gp[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (on) unpack8(*(const uint4*)(a.gamma_p1 + c0), gp);
    uint4 raw[kMaxTopk];
#pragma unroll
    for (int j = 0; j < kMaxTopk; ++j)
        if (j < a.k && on) raw[j] = *(const uint4*)(a.zb + ((size_t)row * a.k + j) * a.P + c0);
    float xg[kMaxTopk][8];
#pragma unroll
    for (int j = 0; j < kMaxTopk; ++j) {
        float ss = 0.f;
        if (j < a.k && on) {
            unpack8(raw[j], xg[j]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                xg[j][i] *= gp[i];
                ss += xg[j][i] * xg[j][i];
            }
        }
        ss = warp_sum(ss);
        if (lane == 0) redk[j][warp] = ss;
    }
    grp_sync(g);
    float mine[kMaxTopk];
    if (t == 0)
        for (int j = 0; j < kMaxTopk; ++j) mine[j] = redk[j][0] + redk[j][1] + redk[j][2] + redk[j][3];
    row_meet(m, row, part, mine, total, 650, g);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < kMaxTopk; ++j)
        if (j < a.k) {
            const float sc = a.w[(size_t)row * a.k + j] * (1.0f / sqrtf(total[j] / (float)a.P + 1e-8f));
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(sc, xg[j][i], acc[i]);
        }
    if (on) *(uint4*)(a.y + (size_t)row * a.P + c0) = pack8(acc);
    grp_sync(g);  // redk / total are free again
}

// ---- the kernel ----------------------------------------------------------------------------------------------------------------
// Trace builds (-DFUSED_TRACE): the first, middle and last CTA stamp the global timer (ns) into u64 words
// [32 + 32 w + slot] (kernel A) or [128 + 32 w + slot] (kernel B) of the status block (w = 0, 1, 2): 0 entry, 1 set-up done, 2 + 4 s: row stage s waits satisfied,
// 3 + 4 s: row stage s done, 4 + 4 s: GEMM stage s epilogue done, 5 + 4 s: stager's wait for stage s satisfied,
// 14 teardown, 15 stage-1 activations staged.
#ifdef FUSED_TRACE
#define FT(slot)                                                                                                  \
    if (a.status != nullptr && (blockIdx.x % 30 == 0 || blockIdx.x == gridDim.x - 1) && blockIdx.x / 30 < 5) {    \
        unsigned long long t_;                                                                                    \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                                   \
        const int w_ = blockIdx.x == gridDim.x - 1 ? 5 : blockIdx.x / 30;                                         \
        ((unsigned long long*)a.status)[32 + (a.row_kind[0] == 3 ? 192 : 0) + 32 * w_ + (slot)] = t_;             \
    }
#else
#define FT(slot)
#endif

__global__ void __launch_bounds__(kDThreads, 1) fused_dense_kernel(const __grid_constant__ FusedArgs a) {
    extern __shared__ unsigned char fused_smem_raw[];
    if (threadIdx.x == 0) { FT(0) }
    const DenseCtx c = dense_setup_cta<kFRing>(fused_smem_raw, a.status);
    if (threadIdx.x == 0) { FT(1) }
    FusedShared& sh = *(FusedShared*)(((uintptr_t)c.extra + 15) & ~(uintptr_t)15);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, cta = blockIdx.x, G = gridDim.x;

    if (warp == 0) {
        if (lane == 0) {
            const uint64_t policy = policy_evict_first();
            uint32_t it = 0;
            for (int s = 0; s < a.n_stages; ++s)
                if (!dense_produce<kFRing>(a.st[s], c, plan_of(a.st[s]), it, policy)) break;
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it = 0;
            int i = 0;
            for (int s = 0; s < a.n_stages; ++s)
                if (!dense_mma<kFRing>(a.st[s], c, plan_of(a.st[s]), it, i)) break;
        }
    } else if (warp < 4) {
        griddep_wait();
        const Grp g{tid - 64, 64, 3};
        const unsigned e = *(volatile const unsigned*)a.launches;
        uint32_t it = 0;
        for (int s = 0; s < a.n_stages; ++s) {
            // the rows this stage multiplies: written by the row stage before it (all M rows, one arrival each)
            if (a.row_kind[s] != 0)
                grp_wait_word(a.dep + s, (e + 1) * (unsigned)(a.M * (a.row_kind[s] == 3 ? a.combine_parts : a.norm_parts)), false, a.budget,
                              a.status, 2, 600 + s, g);
            if (tid == 64) { FT(5 + 4 * s) }
            if (!dense_stage_x<kFRing>(a.st[s], c, plan_of(a.st[s]), it, tid - 64)) break;
            if (tid == 64 && s == 1) { FT(15) }
        }
    } else {
        griddep_wait();
        const int q = warp - 4, te = tid - 128;
        const Grp g{te, 128, 2};
        const unsigned e = *(volatile const unsigned*)a.launches;
        const unsigned ex0 = a.wait_flag[0] != nullptr ? *(volatile const unsigned*)a.wait_epoch[0] : 0u;
        const unsigned ex1 = a.wait_flag[1] != nullptr ? *(volatile const unsigned*)a.wait_epoch[1] : 0u;
        int i = 0;
        bool ok = true;
        for (int s = 0; s <= a.n_stages && ok; ++s) {
            // ---- the row stage in front of GEMM stage s (s == n_stages: the one behind the last) ----
            const int kind = a.row_kind[s];
            // norm / combine rows: part p = (row, 1024-column block) on CTA p (the host checks rows x parts <= grid)
            if (kind == 1 && cta < a.M * a.norm_parts) {
                // every tile of the GEMM stage before, from this GPU and from the present peers
                const int prev = s - 1;
                grp_wait_word(a.dep + 3 + prev, (e + 1) * (unsigned)a.tiles0[prev], false, a.budget, a.status, 2, 610 + s, g);
                if (a.wait_flag[prev] != nullptr)
                    grp_wait_word(a.wait_flag[prev], ((prev ? ex1 : ex0) + 1) * a.wait_contrib[prev], true, a.budget, a.status, 1,
                                  a.wait_stage[prev], g);
                if (te == 0) { FT(2 + 4 * s) }
                const RowMeet m1{a.meet_part, a.meet_count, e, a.norm_parts, 4, a.budget, a.status};
                norm_part_g(a.norm, cta / a.norm_parts, cta % a.norm_parts, m1, sh.red, sh.total, g);
                grp_arrive(a.dep + s, g);
            } else if (kind == 3 && cta < a.M * a.combine_parts) {
                grp_xchg_wait(a.combine.wait, g);
                if (te == 0) { FT(2 + 4 * s) }
                const RowMeet m{a.meet_part + 2 * kMaxRows * 8, a.meet_count + 2 * kMaxRows, e, a.combine_parts, kMaxTopk, a.budget, a.status};
                combine_part_g(a.combine, cta / a.combine_parts, cta % a.combine_parts, m, sh.redk, sh.total, g);
                grp_arrive(a.dep + s, g);
            } else if (kind == 2) {
                // top-k: row r on CTA M + r (a warp's work; on CTA r, in front of its pre-expert row, when the grid is small)
                const bool apart = G >= 2 * a.M + 1;
                const int topk_row_of = apart ? cta - a.M : cta;
                if (topk_row_of >= 0 && topk_row_of < a.M) {
                    // The router's tiles are not finished by their contributors (a tile is shared by some twenty CTAs: one
                    // of them summing all partials was the longest chain of the kernel): every top-k CTA sums its own row's
                    // partial logits in slot order, computes the selection scores (sigmoid in f64 rounded to f32, plus the
                    // expert's bias) on all 128 threads and keeps them in shared memory for the selection.
                    const SegGemm& rg = a.st[1].g[1];
                    const Plan rp = plan_of(a.st[1]);
                    float* scores = (float*)sh.cnt;
                    float* bias = (float*)sh.first;
                    for (int ex = te; ex < a.topk.E; ex += 128) bias[ex] = a.topk.bias[ex];  // in flight during the wait
                    grp_wait_word(a.dep + 2, (e + 1) * (unsigned)a.router_contribs, false, a.budget, a.status, 2, 620, g);
                    const int KSr = stages_of(rg);
                    for (int ex = te; ex < a.topk.E; ex += 128) {
                        const int rt_tile = ex >> 7, col = ex & 127;
                        const uint32_t first = rp.T0 + (uint32_t)rt_tile * KSr;
                        const int n = cta_of(first + KSr - 1, rp.T, rp.G) - cta_of(first, rp.T, rp.G) + 1;
                        const float* src = rg.part + (size_t)rt_tile * rg.maxc * 2048 + topk_row_of * 128 + col;
                        float v = 0.f;
                        int sl = 0;
                        for (; sl + 8 <= n; sl += 8) {
                            float t8[8];
#pragma unroll
                            for (int k = 0; k < 8; ++k) t8[k] = __ldcg(src + (size_t)(sl + k) * 2048);
#pragma unroll
                            for (int k = 0; k < 8; ++k) v += t8[k];
                        }
                        for (; sl < n; ++sl) v += __ldcg(src + (size_t)sl * 2048);
                        a.st[1].f32_out[(size_t)topk_row_of * a.topk.E + ex] = v;
                        scores[ex] = (float)(1.0 / (1.0 + exp(-((double)v * a.topk.mult)))) + bias[ex];
                    }
                    grp_sync(g);
                    if (q == 0) {
                        TopkArgs tk = a.topk;  // the selection reads this row's scores and the biases from shared memory
                        tk.score = scores - (size_t)topk_row_of * a.topk.E;
                        tk.bias = bias;
                        topk_row(tk, topk_row_of, lane, sh.s_ids);
                    }
                    grp_arrive(a.dep + 5, g);
                }
                if (cta == G - 1) {
                    // route tables: every row's top-k (the ids come back from global memory)
                    grp_wait_word(a.dep + 5, (e + 1) * (unsigned)a.M, false, a.budget, a.status, 2, 621, g);
                    if (te == 0) { FT(2 + 4 * s) }
                    for (int i2 = te; i2 < a.M * a.topk.k; i2 += 128) sh.s_ids[i2] = __ldcg(a.topk.ids + i2);
                    grp_sync(g);
                    route_tables(sh.s_ids, a.topk.E, a.b_live * a.topk.k, a.rt, sh.cnt, sh.first, a.topk.e_lo, a.topk.e_hi, g);
                }
                if (cta < a.M) {  // the grid has more than M CTAs (host check): the tables' CTA has no row
                    // pre-expert norm + quantisation: every tile of the pooler, from this GPU and the node's present peers
                    grp_wait_word(a.dep + 4, (e + 1) * (unsigned)a.tiles0[1], false, a.budget, a.status, 2, 630, g);
                    if (a.wait_flag[1] != nullptr)
                        grp_wait_word(a.wait_flag[1], (ex1 + 1) * a.wait_contrib[1], true, a.budget, a.status, 1, a.wait_stage[1], g);
                    if (te == 0) { FT(2 + 4 * s) }
                    nq_row_g(a.nq, cta, sh.red, g, a.status);
                }
            }
            if (te == 0) { FT(3 + 4 * s) }
            if (s == a.n_stages) break;
            // ---- GEMM stage s: finished tiles are announced to the rows that wait for them ----
            TileSignals sg;
            sg.tile_sig[0] = s == 0 ? &a.sig0 : &a.sig1;
            sg.tile_sig[1] = nullptr;
            sg.dep[0] = a.dep + 3 + s;
            sg.dep[1] = a.dep + 2;
            sg.defer1 = a.row_kind[2] == 2;  // kernel A: the router's rows are summed by their top-k CTAs
            ok = dense_epilogue<kFRing>(a.st[s], c, plan_of(a.st[s]), i, q, te, lane, sg);
            if (te == 0) { FT(4 + 4 * s) }
        }
    }
    dense_teardown_cta(c);
    if (tid == 0) { FT(14) }
    // the last CTA out closes the launch: the launch count and the flag block's counts of the exchanges this kernel feeds
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(a.done, 1u) == (unsigned)G - 1) {
            *a.done = 0;
            for (int k = 0; k < 2; ++k)
                if (a.bump_epoch[k] != nullptr) *(volatile unsigned*)a.bump_epoch[k] = *(volatile unsigned*)a.bump_epoch[k] + 1;
            __threadfence();
            atomicAdd(a.launches, 1u);
        }
    }
}

size_t fused_smem() { return DenseLayout<kFRing>::kBytes + sizeof(FusedShared) + 32; }

cudaError_t fused_prepare() {
    return cudaFuncSetAttribute(fused_dense_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fused_smem());
}

cudaError_t fused_launch(const FusedArgs& a, int grid, cudaStream_t s, bool pdl) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kDThreads);
    cfg.dynamicSmemBytes = fused_smem();
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, fused_dense_kernel, a);
}

}  // namespace mk
