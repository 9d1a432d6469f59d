// The kernels around the 62 decoder layers of a verify step: window feeds, the fused entry, the soft cap, and the greedy
// accept that closes a DFlash2 iteration.
//
//   window_feeds   rope rows, int32 cache slots, kv_len and the position -> byte-offset tables of the step
//                  (reference kernels/head.cu:39-110)
//   entry          owner-rank embedding row, weightless embed norm, layer 0's pre-attention norm
//                  (reference kernels/head.cu:112-222, test/reference/muse_spark.py:797-824)
//   softcap        cap tanh(x scale / cap) over the gathered f32 logits (reference kernels/head.cu:234-290)
//   accept         first-arg-max of the soft-capped rows, greedy prefix accept (or the forced table), the step words,
//                  the committed-token ring and the next step's feeds
//                  (reference kernels/dflash/verify_accept.cu:304-400, test/reference/dflash2.py:362-368,649-660)
#include "stages.h"
#include "draft.h"

namespace mk {

// ---- window feeds -------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) window_feeds_kernel(const FeedsArgs a) {
    griddep_wait();
    const int tid = threadIdx.x;
    if (blockIdx.x == 0) {
        if (a.cos_sin_cache != nullptr) {
            for (int i = tid; i < a.rows * a.head_dim; i += 256) {
                const int t = i / a.head_dim, c = i - t * a.head_dim;
                long long pos = a.positions[t];
                if (pos < 0 || pos >= a.cos_sin_rows) {  // no trap: record and clamp
                    if (a.status) a.status[0] = 4, a.status[1] = 300, a.status[3] = (int)pos;
                    pos = 0;
                }
                a.cos_sin[i] = a.cos_sin_cache[pos * a.head_dim + c];
            }
        }
        for (int t = tid; t < a.rows; t += 256) {
            a.loc_full[t] = (int)a.out_cache_loc[t];
            if (a.swa_out_cache_loc != nullptr) a.loc_swa[t] = (int)a.swa_out_cache_loc[t];
        }
        if (tid == 0) a.kv_len[0] = (int)(a.seq_lens[0] + a.rows);
    }
    long long req = a.req_pool_indices[0];
    if (req < 0 || req >= a.r2t_rows) {
        if (tid == 0 && blockIdx.x == 0 && a.status) a.status[0] = 4, a.status[1] = 301, a.status[3] = (int)req;
        req = 0;
    }
    const int* row = a.req_to_token + req * a.r2t_width;
    for (long long j = (long long)blockIdx.x * 256 + tid; j < a.r2t_width; j += (long long)gridDim.x * 256) {
        const long long r = row[j];
        a.pt_full[j] = r * a.kv_row_bytes;
        if (a.full_to_swa != nullptr) {
            long long idx = r < 0 ? r + a.swa_map_len : r;  // a negative index wraps to the appended sentinel row
            if (idx < 0 || idx >= a.swa_map_len) idx = 0;
            a.pt_swa[j] = (long long)a.full_to_swa[idx] * a.kv_row_bytes;
        }
    }
}

// ---- entry ------------------------------------------------------------------------------------------------------------
// One CTA per window row, hidden / 8 threads, 8 columns per thread.
__global__ void __launch_bounds__(1024) entry_kernel(const EntryArgs a) {
    __shared__ float red[33];
    griddep_wait();
    const int row = blockIdx.x, c0 = threadIdx.x * 8;
    const long long id = a.ids[row];
    const bool hit = id >= 0 && id < a.shard_rows * a.ranks;
    const long long owner = hit ? id / a.shard_rows : 0;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (hit) raw = *(const uint4*)(a.embed[owner] + (id - owner * a.shard_rows) * a.hidden + c0);
    const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float x[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(e[j]);
        x[2 * j] = f.x;
        x[2 * j + 1] = f.y;
        ss += f.x * f.x + f.y * f.y;
    }
    const float rstd0 = 1.0f / sqrtf(block_sum(ss, red) / (float)a.hidden + a.eps_embed);
    ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        x[j] = bf16_round(x[j] * rstd0);
        ss += x[j] * x[j];
    }
    float* res = a.residual + (size_t)row * a.hidden + c0;
    *(float4*)res = make_float4(x[0], x[1], x[2], x[3]);
    *(float4*)(res + 4) = make_float4(x[4], x[5], x[6], x[7]);
    const float rstd1 = 1.0f / sqrtf(block_sum(ss, red) / (float)a.hidden + a.eps_pre);
    const uint4 wraw = *(const uint4*)(a.pre_w + c0);
    const __nv_bfloat162* w = reinterpret_cast<const __nv_bfloat162*>(&wraw);
    uint4 o;
    __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 wf = __bfloat1622float2(w[j]);
        ob[j] = __floats2bfloat162_rn((x[2 * j] * rstd1) * wf.x, (x[2 * j + 1] * rstd1) * wf.y);
    }
    *(uint4*)(a.normed + (size_t)row * a.hidden + c0) = o;
}

// ---- soft cap ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) softcap_kernel(const SoftcapArgs a) {
    griddep_wait();
    xchg_wait(a.wait);
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < a.numel; i += (long long)gridDim.x * 256)
        a.out[i] = tanhf((a.x[i] * a.scale) / a.cap) * a.cap;
}

// ---- greedy accept ------------------------------------------------------------------------------------------------------
// Order of the arg-max: the first NaN if the row has one, else the largest value, the lower id on ties (torch.argmax).
struct Best {
    float v;
    int id;
    int nan;
};
__device__ __forceinline__ bool better(const Best& a, const Best& b) {  // a beats b
    if (a.nan != b.nan) return a.nan > b.nan;
    if (a.nan) return a.id < b.id;
    if (a.v != b.v) return a.v > b.v;
    return a.id < b.id;
}
__device__ __forceinline__ Best shfl_best(const Best& x, int o) {
    Best r;
    r.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    r.id = __shfl_xor_sync(0xffffffffu, x.id, o);
    r.nan = __shfl_xor_sync(0xffffffffu, x.nan, o);
    return r;
}

// The end of an iteration, by every thread of one CTA of 1024: `acc` drafts accepted and the bonus token -> the step words
// and the committed-token ring (one thread), then the next iteration's target and draft feeds (all threads).
__device__ __forceinline__ void commit_and_feed(const AcceptArgs& a, int acc, long long bonus) {
    __shared__ long long s_cc, s_p;
    const int tid = threadIdx.x;
    if (tid == 0) {
        const long long p = a.words[0], iter = a.words[4], cnt = a.words[5];
        const long long cc = acc + 1;
        // the accepted drafts: rows 1 .. acc of a chain, the accepted path's rows of a tree
        for (int j = 0; j < acc; ++j) a.out_ring[(cnt + j) % a.ring] = (int)a.tokens[a.tree != nullptr ? a.tree[kTreePath + j + 1] : j + 1];
        a.out_ring[(cnt + acc) % a.ring] = (int)bonus;
        a.words[0] = p + cc;   // P: committed length
        a.words[1] = bonus;    // ANCHOR: next block's row 0
        a.words[2] = acc;      // ACCEPT
        a.words[3] = cc;       // COMMIT
        a.words[4] = iter + 1; // ITER
        a.words[5] = cnt + cc; // OUT_COUNT
        s_cc = cc;
        s_p = p;
    }
    __syncthreads();
    const long long cc = s_cc;
    long long pn = s_p + cc;
    if (a.pool_rows > 0 && pn + a.rows > a.pool_rows) {  // the next window would leave the pools: clamp and record
        if (tid == 0 && a.status != nullptr && atomicCAS(a.status, 0, 4) == 0) a.status[1] = 320, a.status[3] = (int)pn;
        pn = a.pool_rows - a.rows;
    }
    // target feeds: the window's rows sit at positions P' .. P' + rows - 1, identity slots
    if (a.cos_sin != nullptr) {
        for (int i = tid; i < a.rows * 64; i += 1024) {
            const long long pos = min(pn + i / 64, a.cos_sin_rows - 1);
            a.cos_sin[i] = a.cos_sin_cache[pos * 64 + (i & 63)];
        }
    }
    if (tid < a.rows) {
        if (a.loc_full) a.loc_full[tid] = (int)(pn + tid);
        if (a.loc_swa) a.loc_swa[tid] = (int)(pn + tid);
    }
    if (tid == 0 && a.kv_len) a.kv_len[0] = (int)(pn + a.rows);
    // draft feeds: rows [0, B) the block at P' .., rows [B, 2B) the committed context at P' - c' .. (then masked:
    // slot -1, rope row P'); slot = position mod the ring; kv_len = P' + B
    if (a.dslot != nullptr) {
        const int B = a.b_live;
        for (int i = tid; i < 2 * B * 128; i += 1024) {
            const int q = i / 128;
            const bool live = q < B || q - B < cc;
            const long long pq = q < B ? pn + q : pn - cc + q - B;
            const long long r = min(live ? pq : pn, a.dcos_sin_rows - 1);
            if (a.dcos_sin) a.dcos_sin[i] = a.dcos_sin_cache[r * 128 + (i & 127)];
        }
        if (tid < 2 * B) {
            const int q = tid;
            const bool live = q < B || q - B < cc;
            const long long pq = q < B ? pn + q : pn - cc + q - B;
            a.dslot[q] = live ? (int)(pq % a.dring) : -1;
        }
        if (tid == 0) a.dkv_len[0] = (int)(pn + B);
    }
}

// grid = (window rows, kAcceptChunks), 1024 threads: a CTA takes the arg-max of the soft-capped logits over its eighth of
// the row (one CTA a row spent 70 us on 16 SMs walking 202,048 tanh values a row), leaves it in the scratch behind the
// counter and takes the row's ticket; the CTA that completes a row merges the chunks' winners (a total order: the merge
// equals one walk over the row), and the last row to complete runs the accept.
// Scratch words behind `counter[0]`: [1, 1 + rows) the rows' tickets, [64 + 3 (row kAcceptChunks + chunk) ..) the winners.
constexpr int kAcceptChunks = 8;

__global__ void __launch_bounds__(1024) accept_kernel(const AcceptArgs a) {
    __shared__ Best sb[32];
    __shared__ int s_last, s_acc;
    __shared__ long long s_bonus;
    griddep_wait();
    xchg_wait(a.wait);
    const int row = blockIdx.x, chunk = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = a.logits + (size_t)row * a.vocab;
    const int per = (a.vocab + kAcceptChunks - 1) / kAcceptChunks, j0 = chunk * per, j1 = min(a.vocab, j0 + per);
    Best best{-INFINITY, 0x7fffffff, 0};
    for (int j = j0 + tid; j < j1; j += 1024) {
        const float t = tanhf((x[j] * a.scale) / a.cap) * a.cap;
        const Best c{t, j, t != t ? 1 : 0};
        if (better(c, best)) best = c;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const Best c = shfl_best(best, o);
        if (better(c, best)) best = c;
    }
    if (lane == 0) sb[warp] = best;
    __syncthreads();
    if (warp == 0) {
        best = sb[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const Best c = shfl_best(best, o);
            if (better(c, best)) best = c;
        }
        int last = 0;
        if (lane == 0) {
            unsigned* winners = a.counter + 64;
            unsigned* mine = winners + 3 * (row * kAcceptChunks + chunk);
            mine[0] = __float_as_uint(best.v);
            mine[1] = (unsigned)best.id;
            mine[2] = (unsigned)best.nan;
            __threadfence();
            if (atomicInc(a.counter + 1 + row, kAcceptChunks - 1) == kAcceptChunks - 1) {  // the row is complete
                __threadfence();
                for (int k = 0; k < kAcceptChunks; ++k) {
                    const unsigned* w = winners + 3 * (row * kAcceptChunks + k);
                    const Best c{__uint_as_float(__ldcg(w)), (int)__ldcg(w + 1), (int)__ldcg(w + 2)};
                    if (k == 0 || better(c, best)) best = c;
                }
                a.top1[row] = best.id;
                __threadfence();
                const unsigned old = atomicAdd(a.counter, 1u);
                last = old == (unsigned)(gridDim.x - 1);
                if (last) *a.counter = 0;
            }
            s_last = last;
        }
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // ---- the accept (one thread), then the next iteration's feeds (all threads) ----
    if (tid == 0 && a.tree != nullptr) {
        // The token tree's accept (test/reference/dflash2.py:1375-1391): a row matches when its token is the target's
        // arg-max at its parent; it is accepted when it and all its ancestors match; the rows are in preorder, so the
        // accepted path's leaf is the largest accepted row. The forced table names the leaf row instead.
        const long long iter = a.words[4];
        unsigned match = 1u;
        for (int r = 1; r < a.b_live; ++r)
            if (a.tokens[r] == (long long)__ldcg(a.top1 + a.tree[kTreeParent + r])) match |= 1u << r;
        int leaf = 0;
        for (int r = 1; r < a.b_live; ++r)
            if (((unsigned)a.tree[kTreeMask + r] & ~match) == 0u) leaf = r;
        if (a.accept_override != nullptr) {
            const int f = a.accept_override[iter % a.n_override];
            leaf = f < 0 ? 0 : min(f, a.b_live - 1);
        }
        const unsigned on = (unsigned)a.tree[kTreeMask + leaf];
        int n = 0;
        for (int r = 1; r < a.b_live; ++r)
            if ((on >> r) & 1u) a.tree[kTreePath + ++n] = r;  // the window rows at depths 1 .. n
        a.tree[kTreePath] = n;
        s_acc = n;
        s_bonus = __ldcg(a.top1 + leaf);
    } else if (tid == 0) {
        const long long iter = a.words[4];
        int acc = 0;
        while (acc + 1 < a.b_live && a.tokens[acc + 1] == (long long)__ldcg(a.top1 + acc)) ++acc;
        if (a.accept_override != nullptr) {
            const int f = a.accept_override[iter % a.n_override];
            acc = f < 0 ? 0 : min(f, a.b_live - 1);
        }
        s_acc = acc;
        s_bonus = __ldcg(a.top1 + acc);
    }
    __syncthreads();
    commit_and_feed(a, s_acc, s_bonus);
}

// ---- sampled accept -------------------------------------------------------------------------------------------------------
// (test/reference/dflash2.py:703-791) Row r's sampling distribution P_r = softmax(f32(capped logit / T)) over the row's
// top_k largest values (everything equal to the k-th stays), cut to the top-p set (a value stays while the mass of the
// strictly larger values is below top_p), renormalised; then block verification (arXiv:2403.10444, Algorithm 2) or the
// token-by-token test against the walk's probabilities, and the bonus token from the residual max(s P_a - Q_a, 0) (P_a
// after a full accept) by inverse CDF in vocabulary order. Uniforms: Philox, purpose 1, coin e - 1 for prefix e, 15 for
// the bonus. Sums are f64; the selections are exact bisections over the order-preserving 32-bit image of the f32 values.
constexpr int kTopCand = 16;  // candidates per draft slot
#ifdef SAMPLE_TRACE
// trace builds: the global timer at the stages of the sampled accept, as f64 nanoseconds in sample_out[2 + slot]
#define SAMPLE_STAMP(a, slot, who)                                                  \
    if ((who) && threadIdx.x == 0 && (a).sample_out != nullptr) {                    \
        unsigned long long t_;                                                      \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                      \
        (a).sample_out[2 + (slot)] = (double)t_;                                    \
    }
#else
#define SAMPLE_STAMP(a, slot, who)
#endif
__device__ __forceinline__ unsigned ord_key(float v) {
    const unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
// Sums of all threads' values (every thread gets the total). red: 33 slots.
__device__ __forceinline__ double block_sum_d(double v, double* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        double t = lane < (int)(blockDim.x >> 5) ? red[lane] : 0.0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// The last CTA of a sampled accept, all 1024 threads: verification by one thread, the bonus by inverse CDF over the
// accepted row's distribution (a contiguous run of ids per thread), then the step words and the feeds.
__device__ __noinline__ void sample_tail(const AcceptArgs& a) {
    __shared__ double s_scan[1024];
    __shared__ double s_pc[kMaxRows][kTopCand];  // P_e at slot e's candidates
    __shared__ float s_qc[kMaxRows][kTopCand];   // the walk's probabilities
    __shared__ long long s_cd[kMaxRows][kTopCand];
    __shared__ double s_pd[kMaxRows], s_z[kMaxRows];
    __shared__ long long s_tok[kMaxRows + 1];
    __shared__ float s_u[16];
    __shared__ double s_w[32];
    __shared__ int s_acc, s_hit, s_hitw;
    __shared__ long long s_bonus;
    __shared__ double s_scale, s_mass, s_target;
    const int tid = threadIdx.x, V = a.vocab;
    const int gamma = a.b_live - 1;
    SAMPLE_STAMP(a, 5, true)
    // ---- everything the verification reads, fetched by many threads at once ----
    if (tid < a.b_live) {
        s_z[tid] = __ldcg(a.row_z + tid);
        s_tok[tid] = a.tokens[tid];
    }
    if (tid < 16)
        s_u[tid] = philox_uniform((unsigned long long)a.samp[0], (unsigned)a.samp[1], (unsigned)a.words[4], 1u, tid);
    __syncthreads();
    if (tid < gamma * kTopCand) {
        const int e = tid / kTopCand, c = tid % kTopCand;
        const long long id = a.cand[tid];
        s_cd[e][c] = id;
        s_qc[e][c] = a.walk_q[tid];
        s_pc[e][c] = id >= 0 && id < V ? __ldcg(a.es + (size_t)e * V + id) / s_z[e] : 0.0;
    } else if (tid >= 512 && tid < 512 + gamma) {
        const int e = tid - 512;
        const long long d = s_tok[e + 1];
        s_pd[e] = d >= 0 && d < V ? __ldcg(a.es + (size_t)e * V + d) / s_z[e] : 0.0;
    }
    __syncthreads();
    // ---- verification (one thread, shared memory only) ----
    if (tid == 0) {
        double q_d[kMaxRows], ratio[kMaxRows + 1];
        for (int e = 0; e < gamma; ++e) {
            double q = 0.0;
            for (int c = 0; c < kTopCand; ++c)
                if (s_cd[e][c] == s_tok[e + 1]) q += (double)s_qc[e][c];
            q_d[e] = q;
        }
        int acc = 0;
        double scale = 1.0, mass = -1.0;
        if (a.block_verify) {
            ratio[0] = 1.0;
            for (int e = 0; e < gamma; ++e)
                ratio[e + 1] = (q_d[e] > 0.0 && q_d[e] <= 1.0) ? fmin(ratio[e] * s_pd[e] / q_d[e], 1.0) : 0.0;
            for (int e = gamma; e > 0; --e) {
                const double coin = (double)s_u[e - 1];
                if (!(coin < ratio[e])) continue;
                double bar = ratio[e], m = -1.0;
                if (e < gamma && ratio[e] > 0.0 && ratio[e] < 1.0) {
                    // mass of max(r P_e - Q_e, 0): Q_e lives on the slot's candidates only
                    double pc = 0.0, over = 0.0;
                    for (int c = 0; c < kTopCand; ++c) {
                        pc += s_pc[e][c];
                        over += fmax(ratio[e] * s_pc[e][c] - (double)s_qc[e][c], 0.0);
                    }
                    m = ratio[e] * fmax(1.0 - pc, 0.0) + over;
                    bar = m / (m + 1.0 - ratio[e]);
                }
                if (coin < bar) {
                    acc = e;
                    scale = ratio[e];
                    mass = m;
                    break;
                }
            }
        } else {
            while (acc < gamma && q_d[acc] > 0.0 && q_d[acc] <= 1.0 && (double)s_u[acc] * q_d[acc] < s_pd[acc]) ++acc;
        }
        if (a.accept_override != nullptr) {
            const int f = a.accept_override[a.words[4] % a.n_override];
            acc = f < 0 ? 0 : min(f, gamma);
            scale = 1.0;
            mass = -1.0;
        }
        s_acc = acc;
        s_scale = scale;
        s_mass = mass;
    }
    __syncthreads();
    SAMPLE_STAMP(a, 6, true)
    // ---- the bonus: inverse CDF of max(s P_a - Q_a, 0) in vocabulary order; every thread sums a contiguous run of ids
    // (the candidates' share taken off afterwards: max(sP - q, 0) = sP - min(q, sP)) ----
    const int acc = s_acc;
    const bool resid = acc < gamma;
    const double mul = s_scale / s_z[acc];
    const double* es = a.es + (size_t)acc * V;
    const int lane = tid & 31, warp = tid >> 5;
    auto dist = [&](int id) {
        double v = s_scale * (__ldcg(es + id) / s_z[acc]);
        if (resid) {
            for (int c = 0; c < kTopCand; ++c)
                if (s_cd[acc][c] == (long long)id) v -= (double)s_qc[acc][c];
            v = fmax(v, 0.0);
        }
        return v;
    };
    // level 1: a contiguous run of ids per warp, lanes interleaved (coalesced); the candidates' share is taken off the
    // run's total afterwards: max(sP - q, 0) = sP - min(q, sP)
    const int R = (V + 31) / 32, lo1 = min(warp * R, V), hi1 = min(lo1 + R, V);
    {
        double m[8] = {0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0};
        for (int jb = lo1 + lane; jb < hi1; jb += 256) {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int jj = jb + 32 * u;
                if (jj < hi1) m[u] += __ldcg(es + jj);
            }
        }
        double tot = ((m[0] + m[1]) + (m[2] + m[3])) + ((m[4] + m[5]) + (m[6] + m[7]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
        tot *= mul;
        if (resid)
            for (int c = 0; c < kTopCand; ++c) {
                const long long id = s_cd[acc][c];
                if (id >= lo1 && id < hi1) tot -= fmin((double)s_qc[acc][c], s_scale * s_pc[acc][c]);
            }
        if (lane == 0) s_w[warp] = fmax(tot, 0.0);
    }
    __syncthreads();
    if (warp == 0) {
        double incl = s_w[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const double t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        const double total = __shfl_sync(0xffffffffu, incl, 31);
        const double mass = s_mass >= 0.0 ? s_mass : total;
        const double target = (double)s_u[15] * mass;
        const unsigned past = __ballot_sync(0xffffffffu, incl > target);
        s_w[lane] = incl;
        if (lane == 0) {
            s_mass = mass;
            s_target = target;
            s_bonus = V - 1;
            s_hitw = past ? __ffs(past) - 1 : 32;
            s_hit = 1024;
        }
    }
    __syncthreads();
    const double target = s_target;
    if (s_hitw < 32) {
        // level 2: the run that holds the target, a short contiguous piece per thread
        const int hw = s_hitw, lo = min(hw * R, V), hi = min(lo + R, V);
        const double base = hw > 0 ? s_w[hw - 1] : 0.0;
        const int per = (hi - lo + 1023) / 1024, j0 = min(lo + tid * per, hi), j1 = min(j0 + per, hi);
        double mine = 0.0;
        for (int jj = j0; jj < j1; ++jj) mine += dist(jj);
        s_scan[tid] = mine;
        __syncthreads();
        if (tid < 32) {  // running sums of the 1024 pieces: 32 per lane, then across the lanes
            double run = 0.0;
            for (int t = 0; t < 32; ++t) {
                run += s_scan[tid * 32 + t];
                s_scan[tid * 32 + t] = run;
            }
            double incl = run;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const double t = __shfl_up_sync(0xffffffffu, incl, o);
                if (tid >= o) incl += t;
            }
            const double before = base + incl - run;
            for (int t = 0; t < 32; ++t) s_scan[tid * 32 + t] += before;
        }
        __syncthreads();
        if (s_scan[tid] > target && (tid == 0 ? !(base > target) : !(s_scan[tid - 1] > target))) s_hit = tid;
        __syncthreads();
        if (s_hit == 1024 && tid == 0) s_bonus = hi - 1;  // rounding left the target just past the run's own sums
        if (s_hit == tid) {
            double run = tid > 0 ? s_scan[tid - 1] : base;
            long long id = j1 - 1;
            for (int jj = j0; jj < j1; ++jj) {
                run += dist(jj);
                if (run > target) {
                    id = jj;
                    break;
                }
            }
            s_bonus = id;
        }
    }
    __syncthreads();
    if (tid == 0 && a.sample_out != nullptr) {
        a.sample_out[0] = s_scale;
        a.sample_out[1] = s_mass;
    }
    SAMPLE_STAMP(a, 7, true)
    commit_and_feed(a, acc, s_bonus);
    SAMPLE_STAMP(a, 8, true)
}

// grid = window rows, 1024 threads: every live row's distribution; the last CTA to finish verifies and draws the bonus.
__global__ void __launch_bounds__(1024) sample_accept_kernel(const AcceptArgs a) {
    __shared__ double red[33];
    __shared__ float s_mx[32];
    __shared__ int s_last;
    griddep_wait();
    xchg_wait(a.wait);
    const int row = blockIdx.x, tid = threadIdx.x, V = a.vocab;
    const float T = fmaxf(__uint_as_float((unsigned)((unsigned long long)a.samp[3] & 0xFFFFFFFFull)), 1e-5f);
    const float top_p = __uint_as_float((unsigned)((unsigned long long)a.samp[3] >> 32));
    const long long top_k = a.samp[2];
    if (row < a.b_live) {
        const float* x = a.logits + (size_t)row * V;
        float* ys = a.ys + (size_t)row * V;
        double* es = a.es + (size_t)row * V;
        // y = f32(capped logit / T) and the row's largest value
        float mx = -INFINITY;
        for (int j = tid; j < V; j += 1024) {
            const float y = __fdiv_rn(tanhf((x[j] * a.scale) / a.cap) * a.cap, T);
            ys[j] = y;
            mx = fmaxf(mx, y);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if ((tid & 31) == 0) s_mx[tid >> 5] = mx;
        __syncthreads();
        mx = s_mx[0];
        for (int w = 1; w < 32; ++w) mx = fmaxf(mx, s_mx[w]);
        // the k-th largest value: the smallest key t with fewer than k keys above it
        unsigned floor_key = 0u;
        if (top_k < (long long)V) {
            unsigned lo = 0u, hi = 0xFFFFFFFFu;
            while (lo < hi) {
                const unsigned mid = lo + ((hi - lo) >> 1);
                double c = 0.0;
                for (int j = tid; j < V; j += 1024) c += ord_key(ys[j]) > mid ? 1.0 : 0.0;
                if (block_sum_d(c, red) < (double)top_k) hi = mid;
                else lo = mid + 1u;
            }
            floor_key = lo;
        }
        // e = exp(y - max) over the top-k set and its mass
        double z = 0.0;
        for (int j = tid; j < V; j += 1024) {
            const float y = ys[j];
            const double e = ord_key(y) >= floor_key ? exp((double)y - (double)mx) : 0.0;
            es[j] = e;
            z += e;
        }
        z = block_sum_d(z, red);
        // the top-p threshold: the smallest key t with the mass above it below top_p z
        if (top_p < 1.0f) {
            const double tau = (double)top_p * z;
            unsigned lo = floor_key, hi = ord_key(mx);
            while (lo < hi) {
                const unsigned mid = lo + ((hi - lo) >> 1);
                double m = 0.0;
                for (int j = tid; j < V; j += 1024) m += ord_key(ys[j]) > mid ? es[j] : 0.0;
                if (block_sum_d(m, red) < tau) hi = mid;
                else lo = mid + 1u;
            }
            double zk = 0.0;
            for (int j = tid; j < V; j += 1024) {
                const double e = ord_key(ys[j]) >= lo ? es[j] : 0.0;
                es[j] = e;
                zk += e;
            }
            z = block_sum_d(zk, red);
        }
        if (tid == 0) a.row_z[row] = z;
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned old = atomicAdd(a.counter, 1u);
        s_last = old == (unsigned)(gridDim.x - 1);
        if (s_last) *a.counter = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    sample_tail(a);
}

// ---- the rows' distributions on clusters --------------------------------------------------------------------------------------
// The same arithmetic as sample_accept_kernel with a row spread over a cluster of kSampleCluster CTAs (four: sixteen
// clusters of eight did not all fit the GPU at once, and the second wave doubled the time) (one vocabulary
// slice each, its keys in shared memory): the sums and counts meet through distributed shared memory, the two selections
// are 8-way section searches: 12 passes over the slice instead of 32.
constexpr int kSampleCluster = 4;
constexpr size_t kSampleMaxSlice = 204 * 1024;  // bytes of keys a CTA holds; larger vocabularies take the one-CTA-per-row kernel
constexpr int kCountWays = 7;   // thresholds per pass of the top-k search (15 measured slower: 9 passes of 17.7 us against 12 of 9.7)
constexpr int kMassWays = 7;    // thresholds per pass of the top-p search (f64 masses)
constexpr int kSampleWays = kCountWays;  // slots of a cluster reduction
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ double ld_cluster_f64(const double* local, unsigned rank) {
    unsigned addr = (unsigned)__cvta_generic_to_shared(local), remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    double v;
    asm volatile("ld.shared::cluster.f64 %0, [%1];" : "=d"(v) : "r"(remote) : "memory");
    return v;
}
// The cluster's totals of N values per thread (or maxima), identical in every thread of every CTA: CTA totals in a slot
// set that alternates between calls, one cluster barrier, then every CTA adds the slots in rank order.
struct ClusterRed {
    double warp[32][kSampleWays];
    double slot[2][kSampleWays];
    double total[kSampleWays];
    int parity;
};
template <int N, bool MAX>
__device__ __forceinline__ void cluster_reduce(double (&v)[N], ClusterRed& r) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int i = 0; i < N; ++i)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const double t = __shfl_xor_sync(0xffffffffu, v[i], o);
            v[i] = MAX ? fmax(v[i], t) : v[i] + t;
        }
    __syncthreads();  // the previous call's totals have been read
    if (lane == 0)
        for (int i = 0; i < N; ++i) r.warp[warp][i] = v[i];
    __syncthreads();
    const int par = r.parity;
    if (threadIdx.x < N) {
        double t = r.warp[0][threadIdx.x];
        for (int w = 1; w < 32; ++w) t = MAX ? fmax(t, r.warp[w][threadIdx.x]) : t + r.warp[w][threadIdx.x];
        r.slot[par][threadIdx.x] = t;
    }
    cluster_sync_all();
    if (threadIdx.x < N) {
        double t = ld_cluster_f64(&r.slot[par][threadIdx.x], 0);
        for (unsigned c = 1; c < (unsigned)kSampleCluster; ++c) {
            const double o = ld_cluster_f64(&r.slot[par][threadIdx.x], c);
            t = MAX ? fmax(t, o) : t + o;
        }
        r.total[threadIdx.x] = t;
    }
    if (threadIdx.x == 0) r.parity = par ^ 1;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] = r.total[i];
}

// The smallest 32-bit t in [lo, hi] for which `below(t)` holds, given that it holds at hi and is monotone; `measure` fills
// the cluster's totals for up to W thresholds at once.
template <int W, typename Measure, typename Below>
__device__ __forceinline__ unsigned section_search(unsigned lo, unsigned hi, Measure measure, Below below) {
    while (lo < hi) {
        unsigned t[W];
        const unsigned span = hi - lo;
        int n;
        if (span <= (unsigned)W) {
            n = (int)span;
            for (int i = 0; i < W; ++i) t[i] = lo + (unsigned)min(i, n - 1);
        } else {
            n = W;
            const unsigned step = span / (unsigned)(W + 1);
            for (int i = 0; i < W; ++i) t[i] = lo + step * (unsigned)(i + 1);
        }
        double m[W];
        measure(t, m);
        int first = n;
        for (int i = n - 1; i >= 0; --i)
            if (below(m[i])) first = i;
        if (first < n) {
            hi = t[first];
            lo = first == 0 ? lo : t[first - 1] + 1u;
        } else {
            lo = t[n - 1] + 1u;
        }
    }
    return lo;
}

// grid = (kSampleCluster, window rows), clusters of kSampleCluster along x, 1024 threads, dynamic shared memory = one
// slice of keys (4 bytes per vocabulary entry of the slice).
__global__ void __launch_bounds__(1024) sample_accept_cluster_kernel(const AcceptArgs a) {
    extern __shared__ __align__(16) unsigned char dyn_keys[];
    __shared__ ClusterRed cr;
    __shared__ int s_last;
    unsigned* keys = (unsigned*)dyn_keys;
    griddep_wait();
    xchg_wait(a.wait);
    const int row = blockIdx.y, tid = threadIdx.x, V = a.vocab;
    const int slice = (V + kSampleCluster - 1) / kSampleCluster, j0 = min((int)blockIdx.x * slice, V), n = min(slice, V - j0);
    const float T = fmaxf(__uint_as_float((unsigned)((unsigned long long)a.samp[3] & 0xFFFFFFFFull)), 1e-5f);
    const float top_p = __uint_as_float((unsigned)((unsigned long long)a.samp[3] >> 32));
    const long long top_k = a.samp[2];
    if (tid == 0) cr.parity = 0;
    __syncthreads();
    const bool first = blockIdx.x == 0 && blockIdx.y == 0;
    SAMPLE_STAMP(a, 0, first)
    if (row < a.b_live) {  // uniform over the cluster
        const float* x = a.logits + (size_t)row * V + j0;
        float* ys = a.ys + (size_t)row * V + j0;
        double* es = a.es + (size_t)row * V + j0;
        double mxd[1] = {-INFINITY};
        for (int i = tid; i < n; i += 4096) {  // four loads in flight
            float v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = i + u * 1024 < n ? __ldg(x + i + u * 1024) : 0.f;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int ii = i + u * 1024;
                if (ii < n) {
                    const float y = __fdiv_rn(tanhf((v[u] * a.scale) / a.cap) * a.cap, T);
                    ys[ii] = y;
                    keys[ii] = ord_key(y);
                    mxd[0] = fmax(mxd[0], (double)y);
                }
            }
        }
        cluster_reduce<1, true>(mxd, cr);
        const double mx = mxd[0];
        SAMPLE_STAMP(a, 1, first)
        unsigned floor_key = 0u;
        if (top_k < (long long)V) {
            floor_key = section_search<kCountWays>(
                0u, 0xFFFFFFFFu,
                [&](const unsigned (&t)[kCountWays], double (&m)[kCountWays]) {
                    int c[kCountWays] = {};
                    for (int i = tid; i < n; i += 1024) {
                        const unsigned k = keys[i];
#pragma unroll
                        for (int w = 0; w < kCountWays; ++w) c[w] += k > t[w];
                    }
#pragma unroll
                    for (int w = 0; w < kCountWays; ++w) m[w] = (double)c[w];
                    cluster_reduce<kCountWays, false>(m, cr);
                },
                [&](double count) { return count < (double)top_k; });
        }
        SAMPLE_STAMP(a, 2, first)
        double zz[1] = {0.0};
        for (int i = tid; i < n; i += 1024) {
            const unsigned k = keys[i];
            const double e = k >= floor_key ? exp((double)ys[i] - mx) : 0.0;
            es[i] = e;
            zz[0] += e;
        }
        cluster_reduce<1, false>(zz, cr);
        double z = zz[0];
        SAMPLE_STAMP(a, 3, first)
        if (top_p < 1.0f) {
            const double tau = (double)top_p * z;
            const unsigned thr = section_search<kMassWays>(
                floor_key, ord_key((float)mx),
                [&](const unsigned (&t)[kMassWays], double (&m)[kMassWays]) {
#pragma unroll
                    for (int w = 0; w < kMassWays; ++w) m[w] = 0.0;
                    for (int i = tid; i < n; i += 4096) {  // four loads in flight
                        double e[4];
                        unsigned k[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int ii = i + u * 1024;
                            e[u] = ii < n ? es[ii] : 0.0;
                            k[u] = ii < n ? keys[ii] : 0u;
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u)
#pragma unroll
                            for (int w = 0; w < kMassWays; ++w) m[w] += k[u] > t[w] ? e[u] : 0.0;
                    }
                    cluster_reduce<kMassWays, false>(m, cr);
                },
                [&](double mass) { return mass < tau; });
            zz[0] = 0.0;
            for (int i = tid; i < n; i += 1024) {
                const double e = keys[i] >= thr ? es[i] : 0.0;
                es[i] = e;
                zz[0] += e;
            }
            cluster_reduce<1, false>(zz, cr);
            z = zz[0];
        }
        if (tid == 0 && blockIdx.x == 0) a.row_z[row] = z;
        SAMPLE_STAMP(a, 4, first)
    }
    cluster_sync_all();  // no CTA leaves while a peer may still read its slots
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned old = atomicAdd(a.counter, 1u);
        s_last = old == (unsigned)(gridDim.x * gridDim.y - 1);
        if (s_last) *a.counter = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    sample_tail(a);
}

// ---- launchers ------------------------------------------------------------------------------------------------------------
template <typename Args>
static cudaError_t launch_ht(void (*kern)(const Args), dim3 grid, dim3 block, cudaStream_t s, bool pdl, const Args& a) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, a);
}

cudaError_t feeds_launch(const FeedsArgs& a, cudaStream_t s, bool pdl) {
    const int grid = (int)((a.r2t_width + 255) / 256);
    return launch_ht(window_feeds_kernel, dim3(grid < 1 ? 1 : grid), dim3(256), s, pdl, a);
}
cudaError_t entry_launch(const EntryArgs& a, cudaStream_t s, bool pdl) {
    return launch_ht(entry_kernel, dim3(a.rows), dim3(a.hidden / 8), s, pdl, a);
}
cudaError_t softcap_launch(const SoftcapArgs& a, cudaStream_t s, bool pdl) {
    long long blocks = (a.numel + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    return launch_ht(softcap_kernel, dim3((unsigned)blocks), dim3(256), s, pdl, a);
}
cudaError_t headtail_prepare() {
    return cudaFuncSetAttribute(sample_accept_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSampleMaxSlice);
}
cudaError_t accept_launch(const AcceptArgs& a, cudaStream_t s, bool pdl) {
    if (a.samp != nullptr) {
        const size_t slice_bytes = ((size_t)a.vocab + kSampleCluster - 1) / kSampleCluster * 4;
        if (slice_bytes > kSampleMaxSlice) return launch_ht(sample_accept_kernel, dim3(a.rows), dim3(1024), s, pdl, a);
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = kSampleCluster;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(kSampleCluster, a.rows);
        cfg.blockDim = dim3(1024);
        cfg.dynamicSmemBytes = slice_bytes;
        cfg.stream = s;
        cfg.attrs = attr;
        cfg.numAttrs = pdl ? 2 : 1;
        return cudaLaunchKernelEx(&cfg, sample_accept_cluster_kernel, a);
    }
    return launch_ht(accept_kernel, dim3(a.rows, kAcceptChunks), dim3(1024), s, pdl, a);
}

}  // namespace mk
