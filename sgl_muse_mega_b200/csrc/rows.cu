// Row kernels of the layer: everything that is not a weight stream. Each works on the window's <= 16 rows in f32 with
// the bf16 rounding points of the reference's contract (test/reference/muse_spark.py:335-435,587-635).
// They are latency bound (16 rows of work), so each is shaped for few dependent memory round trips: 16-byte loads, every
// load of a pass independent of the others, one block-wide reduction per norm.
#include "stages.h"

namespace mk {

static __device__ __forceinline__ float inv_sqrt(float x) { return 1.0f / sqrtf(x); }

static __device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 x = __bfloat1622float2(p[i]);
        f[2 * i] = x.x;
        f[2 * i + 1] = x.y;
    }
}
static __device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 v;
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return v;
}

// ---- all-reduce consume + post norm + gated residual + pre norm ------------------------------------------------------
// mode 0 (post-attention): branch = bf16(sum over ranks of the bf16 partials, rank order, f32); v = branch
// mode 1 (cross-layer):    v = gathered unpooler row x post_w
// stream' = fma(alpha, stream, scaled), normed = bf16((stream' rstd) pre_w)       (muse_spark.py:335-357)
// One CTA per row, H / 8 threads, 8 consecutive columns per thread. (Tried: a row on a cluster of eight CTAs, totals met
// through distributed shared memory. No gain: the kernel is bound by the arrival of its rows, not by one SM's throughput.)
__global__ void __launch_bounds__(1024) resid_norm_kernel(const NormArgs a) {
    __shared__ float red[33];
    const int row = blockIdx.x, c0 = threadIdx.x * 8;
    const size_t off = (size_t)row * a.H + c0;
    // the layer's own weights are in flight while the predecessor still runs, the residual stream while the peers' rows
    // are still on their way
    const float4 al0 = *(const float4*)(a.alpha + c0), al1 = *(const float4*)(a.alpha + c0 + 4);
    const float4 be0 = *(const float4*)(a.beta + c0), be1 = *(const float4*)(a.beta + c0 + 4);
    const uint4 pw_raw = *(const uint4*)(a.pre_w + c0);
    uint4 post_raw = make_uint4(0, 0, 0, 0);
    if (a.mode != 0) post_raw = *(const uint4*)(a.post_w + c0);
    RT(a.mode != 0, 0)
    // packet mode: the rows that arrive are their own dependency (pkt_take_n), everything else this kernel reads was complete
    // before the producer of those rows passed its own wait, so the kernel does not wait for the producer's grid to end
    if (!a.wait.packets) griddep_wait();
    griddep_launch();
    RT(a.mode != 0, 1)
    const float4 s0 = *(const float4*)(a.stream_in + off), s1 = *(const float4*)(a.stream_in + off + 4);
    xchg_wait(a.wait);  // the all-reduce partials (mode 0) or the unpooler gather (mode 1) of every contributing rank
    float v[8];
    if (a.mode == 0) {
        uint4 part[kMaxRanks];
        if (a.wait.packets) {  // every present rank's partial as it arrives; an absent rank's is 0
            pkt_take_n(part, a.ranks, a.wait.present, [&](int r) { return (void*)(a.src + ((size_t)r * a.M + row) * a.H + c0); }, a.wait);
        } else {
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
                if (r < a.ranks) part[r] = *(const uint4*)(a.src + ((size_t)r * a.M + row) * a.H + c0);
        }
        unpack8(part[0], v);
#pragma unroll
        for (int r = 1; r < kMaxRanks; ++r)
            if (r < a.ranks) {
                float f[8];
                unpack8(part[r], f);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] += f[i];
            }
        const uint4 b = pack8(v);
        *(uint4*)(a.branch + off) = b;
        unpack8(b, v);
    } else {
        float w[8];
        uint4 got[1];
        if (a.wait.packets) pkt_take_n(got, 1, pkt_col_present(a.wait, c0) ? 1u : 0u, [&](int) { return (void*)(a.src + off); }, a.wait);
        else got[0] = *(const uint4*)(a.src + off);
        unpack8(got[0], v);
        unpack8(post_raw, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] *= w[i];
    }
    float pw[8];
    unpack8(pw_raw, pw);
    const float st[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const float al[8] = {al0.x, al0.y, al0.z, al0.w, al1.x, al1.y, al1.z, al1.w};
    const float be[8] = {be0.x, be0.y, be0.z, be0.w, be1.x, be1.y, be1.z, be1.w};
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
    const float post_rstd = inv_sqrt(block_sum(ss, red) / (float)a.H + 1e-8f);
    float ns[8];
    ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float scaled = a.mode == 0 ? (be[i] * post_rstd) * v[i] : be[i] * (v[i] * post_rstd);
        ns[i] = fmaf(al[i], st[i], scaled);
        ss += ns[i] * ns[i];
    }
    const float pre_rstd = inv_sqrt(block_sum(ss, red) / (float)a.H + 1e-5f);
    *(float4*)(a.stream_out + off) = make_float4(ns[0], ns[1], ns[2], ns[3]);
    *(float4*)(a.stream_out + off + 4) = make_float4(ns[4], ns[5], ns[6], ns[7]);
    float h[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) h[i] = (ns[i] * pre_rstd) * pw[i];
    const uint4 hb = pack8(h);
    *(uint4*)(a.normed + off) = hb;
    if (a.normed_f32) {
        unpack8(hb, h);
        *(float4*)(a.normed_f32 + off) = make_float4(h[0], h[1], h[2], h[3]);
        *(float4*)(a.normed_f32 + off + 4) = make_float4(h[4], h[5], h[6], h[7]);
    }
    RT(a.mode != 0, 2)
}

// ---- routing (top-k + route tables) and pre-expert norm + quantisation in one launch ---------------------------------------
// Block 0: one warp per row selects the top-k, then the block builds the route tables. Blocks 1..M: one row each of the
// pre-expert norm + dynamic NVFP4 quantisation (independent of the routing).
//
// top-k: s = sigmoid(mult x logit) (f64, rounded to f32), sel = s + bias, k rounds of arg-max with the smaller id winning
// ties, weights = ((sel - bias) / (sum in selection order + 1e-15)) x route_scale          (muse_spark.py:378-404)
// tables: slots of the live rows grouped by expert: active experts ascending, slots of one expert in slot order.
// nq: n = bf16(bf16(x rsqrt(mean x^2 + eps)) gamma); NVFP4: x_scale = max(amax, 1e-10) / 2688, per 16:
// sf = e4m3(max(gamax, 1e-10) / 6 / x_scale), code = e2m1(n / max(sf x_scale, 1e-10))          (muse_spark.py:407-435)
constexpr int kTopkPer = 32;  // E <= 1024

// PER = experts per lane (E <= 32 PER). The k selection rounds run on registers and shuffles only: a lane keeps its experts'
// scores and biases, proposes its best, and the butterfly carries (score, id, bias) of the winner to every lane.
template <int PER>
static __device__ void topk_row_t(const TopkArgs& a, int row, int lane, int* s_ids) {
    float sel[PER], bs[PER];
    bool bad = false;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = lane + 32 * i;
        sel[i] = -INFINITY;
        bs[i] = 0.f;
        if (e < a.E) {
            bs[i] = a.bias[e];
            if (a.score != nullptr) {  // computed by the router GEMM's epilogue (one thread per logit)
                sel[i] = a.score[(size_t)row * a.E + e];
            } else {
                const double z = (double)a.logits[(size_t)row * a.E + e] * a.mult;
                const float s = (float)(1.0 / (1.0 + exp(-z)));
                sel[i] = s + bs[i];
            }
            // a NaN score (non-finite hidden rows upstream) must still leave k distinct, in-range experts: it ranks
            // below every number, the lower id first; the status block records that the row was not routable
            if (!(sel[i] == sel[i])) {
                sel[i] = -3.0e38f;
                bad = true;
            }
            sel[i] = fmaxf(sel[i], -3.0e38f);  // above the -inf that marks "taken" or "no such expert"
        }
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0 && a.status != nullptr && atomicCAS(a.status, 0, 6) == 0) {
        a.status[1] = 6;  // the routing stage
        a.status[2] = row;
    }
    float total = 0.f, mine = 0.f;
    int myid = 0;
    for (int j = 0; j < a.k; ++j) {
        float bv = -INFINITY, bb = 0.f;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int e = lane + 32 * i;
            if (sel[i] > bv) { bv = sel[i]; bi = e; bb = bs[i]; }  // ascending ids per lane: strict > keeps the smaller id
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            const float ob = __shfl_xor_sync(0xffffffffu, bb, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; bb = ob; }
        }
        const float sv = bv - bb;
        total += sv;
        if (lane == j) { mine = sv; myid = bi; }
        if ((bi & 31) == lane) {
#pragma unroll
            for (int i = 0; i < PER; ++i)
                if (i == (bi >> 5)) sel[i] = -INFINITY;
        }
    }
    const float inv = 1.0f / (total + 1e-15f);
    if (lane < a.k) {
        a.ids[(size_t)row * a.k + lane] = myid;
        a.w[(size_t)row * a.k + lane] = (mine * inv) * a.route_scale;
        s_ids[row * a.k + lane] = myid;
    }
}

static __device__ void topk_row(const TopkArgs& a, int row, int lane, int* s_ids) {
    if (a.E <= 256) topk_row_t<8>(a, row, lane, s_ids);
    else if (a.E <= 512) topk_row_t<16>(a, row, lane, s_ids);
    else topk_row_t<kTopkPer>(a, row, lane, s_ids);
}

// e_hi > e_lo: only the slots routed to an expert in [e_lo, e_hi) enter the tables (this rank's whole experts); the
// other slots belong to other ranks.
// `grp`: the threads that build the tables (S <= grp.n): a whole block, or the epilogue warps of a fused kernel.
static __device__ void route_tables(const int* s_ids, int E, int S, RouteTables* rt, int* cnt, int* first, int e_lo, int e_hi,
                                    const Grp& grp) {
    const int tid = grp.tid, nt = grp.n;
    for (int e = tid; e < E; e += nt) cnt[e] = 0;
    grp_sync(grp);
    int my_e = -1;
    if (tid < S) {
        my_e = s_ids[tid];
        if (e_hi > e_lo && (my_e < e_lo || my_e >= e_hi)) my_e = -1;
        if (my_e >= 0) atomicAdd(&cnt[my_e], 1);
    }
    grp_sync(grp);
    if (tid < 32) {
        // exclusive scan of the counts over the experts, 32 experts per step; compaction of the active ones
        int base = 0, nact = 0;
        for (int e0 = 0; e0 < E; e0 += 32) {
            const int e = e0 + tid, c = e < E ? cnt[e] : 0;
            int incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, o);
                if (tid >= o) incl += t;
            }
            const unsigned act = __ballot_sync(0xffffffffu, c > 0);
            if (e < E) first[e] = base + incl - c;
            if (c > 0) {
                const int pos = nact + __popc(act & ((1u << tid) - 1));
                rt->act_e[pos] = e;
                rt->act_off[pos] = base + incl - c;
            }
            base += __shfl_sync(0xffffffffu, incl, 31);
            nact += __popc(act);
        }
        if (tid == 0) {
            rt->act_off[nact] = base;
            rt->n_active = nact;
        }
    }
    grp_sync(grp);
    if (tid < S && my_e >= 0) {
        int before = 0;
        for (int s = 0; s < tid; ++s) before += (s_ids[s] == my_e);
        rt->slot[first[my_e] + before] = tid;
    }
}
static __device__ void route_tables(const int* s_ids, int E, int S, RouteTables* rt, int* cnt, int* first, int e_lo = 0,
                                    int e_hi = 0) {
    route_tables(s_ids, E, S, rt, cnt, first, e_lo, e_hi, block_grp());
}

static __device__ void nq_row(const NqArgs& a, int row, float* red) {
    const int tid = threadIdx.x, nt = blockDim.x;
    const int groups = a.P / 16;
    const bf16* x = a.pooled + (size_t)row * a.P;
    // one 16-element group per thread and pass (P / 16 <= blockDim for P <= 8192)
    float n[16];
    float ss = 0.f;
    const bool own = tid < groups;
    if (own) {
        float g[16];
        if (a.wait.packets) {  // both packets of the group lie in one source's band (bands are multiples of 16 columns)
            uint4 got[2];
            pkt_take_n(got, 2, pkt_col_present(a.wait, tid * 16) ? 3u : 0u, [&](int j) { return (void*)(x + tid * 16 + 8 * j); }, a.wait);
            unpack8(got[0], *(float(*)[8])g);
            unpack8(got[1], *(float(*)[8])(g + 8));
        } else {
            unpack8(*(const uint4*)(x + tid * 16), *(float(*)[8])g);
            unpack8(*(const uint4*)(x + tid * 16 + 8), *(float(*)[8])(g + 8));
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            n[i] = g[i];
            ss += g[i] * g[i];
        }
    }
    (void)nt;
    const float rstd = inv_sqrt(block_sum(ss, red) / (float)a.P + a.eps);
    float gmax = 0.f;
    if (own) {
        float gm[16];
        unpack8(*(const uint4*)(a.gamma + tid * 16), *(float(*)[8])gm);
        unpack8(*(const uint4*)(a.gamma + tid * 16 + 8), *(float(*)[8])(gm + 8));
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            n[i] = bf16_round(bf16_round(n[i] * rstd) * gm[i]);
            gmax = fmaxf(gmax, fabsf(n[i]));
        }
    }
    if (a.bf16_out) {
        if (own) {
            bf16* o = (bf16*)a.q + (size_t)row * a.P + tid * 16;
            *(uint4*)o = pack8(*(float(*)[8])n);
            *(uint4*)(o + 8) = pack8(*(float(*)[8])(n + 8));
        }
        return;
    }
    const float amax = block_max(gmax, red);
    const float kSixth = 1.0f / 6.0f, kInv2688 = 1.0f / 2688.0f;
    const float x_scale = fmaxf(amax, 1e-10f) * kInv2688;
    const float inv_x = 1.0f / x_scale;
    if (tid == 0) a.x_scale[row] = x_scale;
    if (own) {
        const uint32_t sfb = float_to_e4m3((fmaxf(gmax, 1e-10f) * kSixth) * inv_x);
        const float out_scale = 1.0f / fmaxf(e4m3_to_float(sfb) * x_scale, 1e-10f);
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            lo |= float_to_e2m1(n[i] * out_scale) << (4 * i);
            hi |= float_to_e2m1(n[8 + i] * out_scale) << (4 * i);
        }
        *(uint2*)(a.q + (size_t)row * (a.P / 2) + tid * 8) = make_uint2(lo, hi);
        a.sf[(size_t)row * groups + tid] = (unsigned char)sfb;
    }
}

struct RouteNqArgs {
    TopkArgs topk;
    NqArgs nq;
    RouteTables* rt;
    int b_live;
    unsigned* ticket;  // zero between launches: the routing rows' arrivals
};

// Blocks 0 .. M - 1: the routing of one row each - a thread per expert forms the selection score (the f64 sigmoid is the
// long pole: one per thread instead of a row's worth per lane), warp 0 selects the top-k from shared memory, and the row
// takes a ticket; the last row to arrive builds the route tables from every row's ids. Blocks M .. 2 M - 1: the pre-expert
// norm + quantisation of one row each.
__global__ void __launch_bounds__(512) route_nq_kernel(const RouteNqArgs a) {
    __shared__ float red[33];
    __shared__ int s_ids[kMaxSlots];
    __shared__ int cnt[1024];
    __shared__ int first[1024];
    __shared__ float s_sel[1024];
    __shared__ int s_last;
    const int M = a.topk.M, E = a.topk.E, tid = threadIdx.x;
    // the biases do not depend on the predecessor
    float bias[2] = {0.f, 0.f};
    if ((int)blockIdx.x < M) {
#pragma unroll
        for (int r = 0; r < 2; ++r)
            if (tid + 512 * r < E) bias[r] = a.topk.bias[tid + 512 * r];
    }
    RT(2, 0)
    // packet mode: the pooled rows and (where this kernel forms the scores) the router's f32 logits are their own dependency
    const bool polled = a.nq.wait.packets && ((int)blockIdx.x >= M || a.topk.score == nullptr);
    if (!polled) griddep_wait();
    else griddep_launch();
    RT(2, 1)
    if ((int)blockIdx.x >= M) {
        xchg_wait(a.nq.wait);  // the pooler gather of the node's ranks
        nq_row(a.nq, blockIdx.x - M, red);
        RT(2, 2)
        return;
    }
    const int row = blockIdx.x;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int e = tid + 512 * r;
        if (e < E) {
            if (a.topk.score != nullptr) {
                s_sel[e] = a.topk.score[(size_t)row * E + e];
            } else {
                float lg;
                if (a.nq.wait.packets) {  // an f32 of all ones marks a logit that has not arrived (pkt_take_n's rule, 4 bytes)
                    unsigned* p = (unsigned*)(a.topk.logits + (size_t)row * E + e);
                    long long polls = 0;
                    unsigned v;
                    for (;;) {
                        asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
                        if (v != kPktMark || !pkt_again(a.nq.wait, polls)) break;
                    }
                    *p = kPktMark;
                    lg = __uint_as_float(v);
                } else {
                    lg = a.topk.logits[(size_t)row * E + e];
                }
                const double z = (double)lg * a.topk.mult;
                s_sel[e] = (float)(1.0 / (1.0 + exp(-z))) + bias[r];
            }
        }
    }
    __syncthreads();
    if (tid < 32) {
        TopkArgs tk = a.topk;
        tk.score = s_sel - (size_t)row * E;
        topk_row(tk, row, tid, s_ids);
        __threadfence();  // the row's ids and weights, then its arrival
        __syncwarp();
        if (tid == 0) s_last = atomicInc(a.ticket, (unsigned)(M - 1)) == (unsigned)(M - 1);
    }
    __syncthreads();
    RT(2, 2)
    if (!s_last) return;
    __threadfence();
    const int S = M * a.topk.k;
    for (int i = tid; i < S; i += 512) s_ids[i] = __ldcg(a.topk.ids + i);
    __syncthreads();
    route_tables(s_ids, E, a.b_live * a.topk.k, a.rt, cnt, first, a.topk.e_lo, a.topk.e_hi);
    RT(2, 3)
}

// ---- h row view: scales moved to the row's largest exponent ---------------------------------------------------------------
// e_row = max over the full row's group exponents; sf' = sf x 2^-(e_row - e): exponent-field move while normal, round half
// up on the subnormal grid                                                                 (muse_spark.py:447-491)
__global__ void __launch_bounds__(256) hrow_kernel(const unsigned char* z_sf, const signed char* z_ex, int groups, int slots_live,
                                                   unsigned char* z_sfd, float* rowscale, const XchgWait wait) {
    __shared__ float red[33];
    griddep_wait();
    griddep_launch();
    xchg_wait(wait);  // every rank's column band of the h planes
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
// One CTA per row, P / 8 threads, 8 columns per thread; the k slot rows are read once and stay in registers.
constexpr int kMaxTopk = 8;

__global__ void __launch_bounds__(512) combine_kernel(const CombineArgs a) {
    __shared__ float red[kMaxTopk][17];
    __shared__ float sc[kMaxTopk];
    const int row = blockIdx.x, tid = threadIdx.x, c0 = tid * 8, warp = tid >> 5, lane = tid & 31;
    const int nw = blockDim.x >> 5;
    const uint4 gp_raw = *(const uint4*)(a.gamma_p1 + c0);  // a weight: in flight while the predecessor still runs
    // the row's routing weights were written before g1 ran: requested here too (a pad row has none)
    float w_pre = 0.f;
    if (tid < kMaxTopk && tid < a.k && row < a.b_live) w_pre = a.w[(size_t)row * a.k + tid];
    RT(4, 0)
    // (packet mode, as the norms: no wait for g2's grid. With polls that slept 32 ns between rounds this lost 3.8 us: the
    // CTAs take the first SMs g2 frees and poll through g2's last 10 us, and a sleeping poll noticed the last rows late.)
    if (!a.wait.packets) griddep_wait();
    else griddep_launch();
    RT(4, 1)
    xchg_wait(a.wait);  // every rank's column band of the expert outputs
    if (row >= a.b_live) {
        *(uint4*)(a.y + (size_t)row * a.P + c0) = make_uint4(0, 0, 0, 0);
        return;
    }
    float gp[8];
    unpack8(gp_raw, gp);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j0 = 0; j0 < a.k; j0 += kMaxTopk) {
        const int kk = min(kMaxTopk, a.k - j0);
        uint4 raw[kMaxTopk];
        if (a.wait.packets) {
            pkt_take_n(raw, kk, pkt_col_present(a.wait, c0) ? 0xFFu : 0u,
                       [&](int j) { return (void*)(a.zb + ((size_t)row * a.k + j0 + j) * a.P + c0); }, a.wait);
        } else {
#pragma unroll
            for (int j = 0; j < kMaxTopk; ++j)
                if (j < kk) raw[j] = *(const uint4*)(a.zb + ((size_t)row * a.k + j0 + j) * a.P + c0);
        }
        float xg[kMaxTopk][8];
#pragma unroll
        for (int j = 0; j < kMaxTopk; ++j) {
            float ss = 0.f;
            if (j < kk) {
                unpack8(raw[j], xg[j]);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    xg[j][i] *= gp[i];
                    ss += xg[j][i] * xg[j][i];
                }
            }
            ss = warp_sum(ss);
            if (lane == 0) red[j][warp] = ss;
        }
        __syncthreads();
        if (tid < kMaxTopk && tid < kk) {
            float s = 0.f;
            for (int w = 0; w < nw; ++w) s += red[tid][w];
            const float wj = j0 == 0 ? w_pre : a.w[(size_t)row * a.k + j0 + tid];
            sc[tid] = wj * (1.0f / sqrtf(s / (float)a.P + 1e-8f));
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
    *(uint4*)(a.y + (size_t)row * a.P + c0) = pack8(acc);
    RT(4, 2)
}

// ---- qkv row ops: qk norm, q scale, interleaved-pair RoPE, KV append -----------------------------------------------------------
// One warp per (row, head) over the q, k and v heads of the bf16 qkv row                    (muse_spark.py:601-635)
__global__ void __launch_bounds__(256) rowops_kernel(const RowopsArgs a) {
    griddep_wait();
    griddep_launch();
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

}  // namespace mk

#include "segments.cuh"
#include "fused.cuh"

namespace mk {

// ---- launch helpers -----------------------------------------------------------------------------------------------------------

template <typename... KArgs, typename... Args>
static cudaError_t launch1(void (*kern)(KArgs...), dim3 grid, dim3 block, cudaStream_t stream, bool pdl, Args... args) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

cudaError_t resid_norm_launch(const NormArgs& a, cudaStream_t s, bool pdl) {
    return launch1(resid_norm_kernel, dim3(a.M), dim3(a.H / 8), s, pdl, a);
}
cudaError_t route_nq_launch(const TopkArgs& t, const NqArgs& n, RouteTables* rt, int b_live, unsigned* ticket, cudaStream_t s,
                            bool pdl) {
    RouteNqArgs a{t, n, rt, b_live, ticket};
    return launch1(route_nq_kernel, dim3(2 * t.M), dim3(512), s, pdl, a);
}
cudaError_t hrow_launch(const unsigned char* z_sf, const signed char* z_ex, int groups, int slots_live, int slots,
                        unsigned char* z_sfd, float* rowscale, const XchgWait& wait, cudaStream_t s, bool pdl) {
    return launch1(hrow_kernel, dim3(slots), dim3(256), s, pdl, z_sf, z_ex, groups, slots_live, z_sfd, rowscale, wait);
}
cudaError_t combine_launch(const CombineArgs& a, int M, cudaStream_t s, bool pdl) {
    return launch1(combine_kernel, dim3(M), dim3(a.P / 8), s, pdl, a);
}
cudaError_t rowops_launch(const RowopsArgs& a, cudaStream_t s, bool pdl) {
    const int warps = a.M * (a.qh + 2 * a.kvh);
    return launch1(rowops_kernel, dim3((warps + 7) / 8), dim3(256), s, pdl, a);
}

}  // namespace mk

RT_READ(mk_rows_trace_read)
