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

// grid = window rows, 1024 threads: per-row arg-max of the soft-capped logits; the last CTA to finish runs the accept.
__global__ void __launch_bounds__(1024) accept_kernel(const AcceptArgs a) {
    __shared__ Best sb[32];
    __shared__ int s_last;
    __shared__ long long s_cc, s_p;
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
        const long long p = a.words[0], iter = a.words[4], cnt = a.words[5];
        int acc = 0;
        while (acc + 1 < a.b_live && a.tokens[acc + 1] == (long long)__ldcg(a.top1 + acc)) ++acc;
        if (a.accept_override != nullptr) {
            const int f = a.accept_override[iter % a.n_override];
            acc = f < 0 ? 0 : min(f, a.b_live - 1);
        }
        const long long cc = acc + 1, bonus = __ldcg(a.top1 + acc);
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
    return launch_ht(accept_kernel, dim3(a.rows), dim3(1024), s, pdl, a);
}

}  // namespace mk
