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
        for (int j = 0; j < acc; ++j) a.out_ring[(cnt + j) % a.ring] = (int)a.tokens[j + 1];
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

// grid = window rows, 1024 threads: per-row arg-max of the soft-capped logits; the last CTA to finish runs the accept.
__global__ void __launch_bounds__(1024) accept_kernel(const AcceptArgs a) {
    __shared__ Best sb[32];
    __shared__ int s_last, s_acc;
    __shared__ long long s_bonus;
    griddep_wait();
    xchg_wait(a.wait);
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = a.logits + (size_t)row * a.vocab;
    Best best{-INFINITY, 0x7fffffff, 0};
    for (int j = tid; j < a.vocab; j += 1024) {
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
        if (lane == 0) {
            a.top1[row] = best.id;
            __threadfence();
            const unsigned old = atomicAdd(a.counter, 1u);
            s_last = old == (unsigned)(gridDim.x - 1);
            if (s_last) *a.counter = 0;
        }
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // ---- the accept (one thread), then the next iteration's feeds (all threads) ----
    if (tid == 0) {
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

// grid = window rows, 1024 threads: every live row's distribution; the last CTA to finish verifies and draws the bonus.
__global__ void __launch_bounds__(1024) sample_accept_kernel(const AcceptArgs a) {
    __shared__ double red[33];
    __shared__ float s_mx[32];
    __shared__ double s_scan[1024];
    __shared__ int s_last, s_acc, s_hit;
    __shared__ long long s_bonus;
    __shared__ double s_scale, s_mass;
    __shared__ long long s_cand[kTopCand];
    __shared__ float s_q[kTopCand];
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
    // ---- verification (one thread) ----
    const int gamma = a.b_live - 1;
    if (tid == 0) {
        const unsigned long long seed = (unsigned long long)a.samp[0];
        const unsigned stream = (unsigned)a.samp[1], iter = (unsigned)a.words[4];
        double p_d[kMaxRows], q_d[kMaxRows], ratio[kMaxRows + 1];
        for (int e = 0; e < gamma; ++e) {
            const long long d = a.tokens[e + 1];
            p_d[e] = d >= 0 && d < V ? __ldcg(a.es + (size_t)e * V + d) / __ldcg(a.row_z + e) : 0.0;
            double q = 0.0;
            for (int c = 0; c < kTopCand; ++c)
                if (a.cand[e * kTopCand + c] == d) q += (double)a.walk_q[e * kTopCand + c];
            q_d[e] = q;
        }
        int acc = 0;
        double scale = 1.0, mass = -1.0;
        if (a.block_verify) {
            ratio[0] = 1.0;
            for (int e = 0; e < gamma; ++e)
                ratio[e + 1] = (q_d[e] > 0.0 && q_d[e] <= 1.0) ? fmin(ratio[e] * p_d[e] / q_d[e], 1.0) : 0.0;
            for (int e = gamma; e > 0; --e) {
                const double coin = (double)philox_uniform(seed, stream, iter, 1u, e - 1);
                if (!(coin < ratio[e])) continue;
                double bar = ratio[e], m = -1.0;
                if (e < gamma && ratio[e] > 0.0 && ratio[e] < 1.0) {
                    // mass of max(r P_e - Q_e, 0): Q_e lives on the slot's candidates only
                    double pc = 0.0, over = 0.0;
                    for (int c = 0; c < kTopCand; ++c) {
                        const long long id = a.cand[e * kTopCand + c];
                        const double pe = id >= 0 && id < V ? __ldcg(a.es + (size_t)e * V + id) / __ldcg(a.row_z + e) : 0.0;
                        pc += pe;
                        over += fmax(ratio[e] * pe - (double)a.walk_q[e * kTopCand + c], 0.0);
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
            while (acc < gamma && q_d[acc] > 0.0 && q_d[acc] <= 1.0 &&
                   (double)philox_uniform(seed, stream, iter, 1u, acc) * q_d[acc] < p_d[acc])
                ++acc;
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
    // ---- the bonus: inverse CDF of max(s P_a - Q_a, 0) in vocabulary order (all threads, a contiguous run of ids each) ----
    const int acc = s_acc;
    const double scale = s_scale, zr = __ldcg(a.row_z + acc);
    const bool resid = acc < gamma;
    if (tid < kTopCand) {
        s_cand[tid] = resid ? a.cand[acc * kTopCand + tid] : -1;
        s_q[tid] = resid ? a.walk_q[acc * kTopCand + tid] : 0.f;
    }
    __syncthreads();
    const double* es = a.es + (size_t)acc * V;
    const int per = (V + 1023) / 1024, j0 = min(tid * per, V), j1 = min(j0 + per, V);
    auto dist = [&](int j) {
        double v = scale * (__ldcg(es + j) / zr);
        if (resid) {
            for (int c = 0; c < kTopCand; ++c)
                if (s_cand[c] == (long long)j) v -= (double)s_q[c];
            v = fmax(v, 0.0);
        }
        return v;
    };
    double mine = 0.0;
    for (int j = j0; j < j1; ++j) mine += dist(j);
    s_scan[tid] = mine;
    __syncthreads();
    if (tid == 0) {  // running sums of the 1024 runs, in order
        double run = 0.0;
        for (int t = 0; t < 1024; ++t) {
            run += s_scan[t];
            s_scan[t] = run;
        }
        const double total = run, mass = s_mass >= 0.0 ? s_mass : total;
        const double target = (double)philox_uniform((unsigned long long)a.samp[0], (unsigned)a.samp[1], (unsigned)a.words[4], 1u, 15) * mass;
        int hit = -1;
        for (int t = 0; t < 1024 && hit < 0; ++t)
            if (s_scan[t] > target) hit = t;
        s_hit = hit;
        s_mass = mass;
        red[0] = target;
        s_bonus = V - 1;
    }
    __syncthreads();
    if (s_hit == tid) {
        double run = tid > 0 ? s_scan[tid - 1] : 0.0;
        const double target = red[0];
        long long id = j1 - 1;
        for (int j = j0; j < j1; ++j) {
            run += dist(j);
            if (run > target) {
                id = j;
                break;
            }
        }
        s_bonus = id;
    }
    __syncthreads();
    if (tid == 0 && a.sample_out != nullptr) {
        a.sample_out[0] = s_scale;
        a.sample_out[1] = s_mass;
    }
    commit_and_feed(a, acc, s_bonus);
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
cudaError_t accept_launch(const AcceptArgs& a, cudaStream_t s, bool pdl) {
    if (a.samp != nullptr) return launch_ht(sample_accept_kernel, dim3(a.rows), dim3(1024), s, pdl, a);
    return launch_ht(accept_kernel, dim3(a.rows), dim3(1024), s, pdl, a);
}

}  // namespace mk
