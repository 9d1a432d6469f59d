// The DFlash2 token tree: the draft head's tree over its lattice and the compaction of the accepted path.
//
// The verify window's 16 rows form a tree rooted at the anchor instead of a chain. Every lattice row (slot e, predecessor
// candidate p) offers its four best successors with their log-probabilities inside those four (fp32 per operation, exp and
// log evaluated in double and rounded, so the values are the correctly rounded fp32 ones); the tree grows best-first by path
// log-probability (ties: the earlier push) until it has 16 rows; the rows are laid out in preorder, the better-ranked child
// first, so that the accepted path's leaf is the largest accepted row. Arithmetic contract: test/reference/dflash2.py:1295-1372
// (token_tree), reference kernel kernels/dflash/tree.cuh (fan_row, walk, tree_compact).
//
// The table (i32 [kTreeWords]): parent[16] (-1 for the anchor), depth[16], ancestor mask[16] (bit j: row j is the row or one
// of its ancestors), path[16] (written by the tree accept: [0] the accept length, [i] the window row at depth i), then the
// window rows' slots in the full and the sliding-window pools as they were when the tree was made (the accept moves the
// feeds on before the compaction runs).
#include "draft.h"

namespace mk {

namespace {

constexpr int kFan = 4;
constexpr int kFront = 64;  // 4 + 15 x 3 entries at most

struct Offer {
    float lp[kFan];
    int idx[kFan];
};

// The four best of a 16-entry score row (larger first, the smaller index on a tie: torch.argsort stable descending) and
// their log-probabilities inside the four. One warp; lanes 0..15 hold the row.
__device__ __forceinline__ Offer fan_row(const float* row, int lane) {
    float v = lane < 16 ? row[lane] : -INFINITY;
    bool taken = lane >= 16;
    Offer o;
#pragma unroll
    for (int k = 0; k < kFan; ++k) {
        float bv = taken ? -INFINITY : v;
        int bi = taken ? 64 : lane;
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, s);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, s);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        o.lp[k] = bv;
        o.idx[k] = bi;
        if (lane == bi) taken = true;
    }
    const float top = o.lp[0];
    float d[kFan], total = 0.f;
#pragma unroll
    for (int k = 0; k < kFan; ++k) {
        d[k] = __fsub_rn(o.lp[k], top);
        total = __fadd_rn(total, (float)exp((double)d[k]));
    }
    const float lse = (float)log((double)total);
#pragma unroll
    for (int k = 0; k < kFan; ++k) o.lp[k] = __fsub_rn(d[k], lse);
    return o;
}

}  // namespace

// grid 1, 32 threads
__global__ void __launch_bounds__(32) dtree_walk_kernel(const DTreeArgs a) {
    __shared__ float f_lp[kFront];
    __shared__ int f_seq[kFront], f_slot[kFront], f_cand[kFront], f_par[kFront], f_rank[kFront];
    __shared__ int n_slot[kTreeRows], n_cand[kTreeRows], n_par[kTreeRows], n_depth[kTreeRows], n_rank[kTreeRows];
    __shared__ unsigned long long key[kTreeRows];
    griddep_wait();
    const int lane = threadIdx.x, gamma = a.rows - 1;
    int nf = 0, seq = 0, nn = 1;
    if (lane == 0) {
        n_slot[0] = -1; n_cand[0] = 0; n_par[0] = -1; n_depth[0] = 0; n_rank[0] = 0;
    }
    auto push = [&](const Offer& o, float base, bool root, int slot, int par) {
        if (lane == 0) {
            for (int k = 0; k < kFan; ++k) {
                f_lp[nf + k] = root ? o.lp[k] : __fadd_rn(base, o.lp[k]);
                f_seq[nf + k] = seq + k;
                f_slot[nf + k] = slot;
                f_cand[nf + k] = o.idx[k];
                f_par[nf + k] = par;
                f_rank[nf + k] = k + 1;
            }
        }
        nf += kFan;
        seq += kFan;
        __syncwarp();
    };
    push(fan_row(a.scores, lane), 0.f, true, 0, 0);
    while (nn < a.rows) {
        // the frontier's best: the largest path log-probability, the earlier push on a tie
        float bv = -INFINITY;
        int bs = 0x7fffffff, bi = -1;
        for (int i = lane; i < nf; i += 32) {
            const float v = f_lp[i];
            const int s = f_seq[i];
            if (v > bv || (v == bv && s < bs)) { bv = v; bs = s; bi = i; }
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, s);
            const int os = __shfl_xor_sync(0xffffffffu, bs, s), oi = __shfl_xor_sync(0xffffffffu, bi, s);
            if (ov > bv || (ov == bv && os < bs)) { bv = ov; bs = os; bi = oi; }
        }
        const int slot = f_slot[bi], c = f_cand[bi], par = f_par[bi], rank = f_rank[bi];
        __syncwarp();
        if (lane == 0) {
            n_slot[nn] = slot; n_cand[nn] = c; n_par[nn] = par; n_depth[nn] = slot + 1; n_rank[nn] = rank;
            const int last = nf - 1;  // the popped entry's place takes the last entry
            f_lp[bi] = f_lp[last]; f_seq[bi] = f_seq[last]; f_slot[bi] = f_slot[last]; f_cand[bi] = f_cand[last];
            f_par[bi] = f_par[last]; f_rank[bi] = f_rank[last];
        }
        nf -= 1;
        __syncwarp();
        const int me = nn++;
        if (slot + 1 < gamma) push(fan_row(a.scores + ((size_t)(slot + 1) * 16 + c) * 16, lane), bv, false, slot + 1, me);
    }
    __syncwarp();
    // preorder: a row's key holds the ranks along its path, the shallower depth in the higher digits
    if (lane == 0) {
        key[0] = 0;
        for (int r = 1; r < a.rows; ++r) key[r] = key[n_par[r]] | ((unsigned long long)n_rank[r] << (3 * (kTreeRows - 1 - n_depth[r])));
    }
    __syncwarp();
    if (lane < a.rows) {
        int o = 0, po = 0;
        const int par = n_par[lane];
        for (int j = 0; j < a.rows; ++j) {
            o += key[j] < key[lane];
            if (par >= 0) po += key[j] < key[par];
        }
        a.table[kTreeParent + o] = par < 0 ? -1 : po;
        a.table[kTreeDepth + o] = n_depth[lane];
        a.verify_ids[o] = lane == 0 ? a.words[1] : a.cand[(size_t)n_slot[lane] * 16 + n_cand[lane]];
    }
    __syncwarp();
    if (lane == 0) {  // ancestor masks in preorder (a parent precedes its children)
        a.table[kTreeMask + 0] = 1;
        for (int p = 1; p < a.rows; ++p) a.table[kTreeMask + p] = a.table[kTreeMask + a.table[kTreeParent + p]] | (1 << p);
    }
    __syncwarp();
    if (a.cos_sin != nullptr) {  // the window's rotations by depth (the accept wrote a chain's: row r at P + r)
        const long long P = a.words[0];
        for (int i = lane; i < a.rows * 64; i += 32) {
            const long long pos = min(P + a.table[kTreeDepth + i / 64], a.cos_sin_rows - 1);
            a.cos_sin[i] = a.cos_sin_cache[pos * 64 + (i & 63)];
        }
    }
    if (lane < a.rows) {
        a.table[kTreePath + lane] = 0;
        a.table[kTreeSlotFull + lane] = a.loc_full != nullptr ? a.loc_full[lane] : 0;
        a.table[kTreeSlotSwa + lane] = a.loc_swa != nullptr ? a.loc_swa[lane] : 0;
    }
}

// One CTA per K / V pool, kCompactCapCtas per capture buffer (a captured row is tens of KB, a K / V row a few hundred bytes):
// the row at depth i (1 .. accept) takes the bytes the path's row path[i] held before the launch. A source path[i] >= i can be
// a later destination, so a thread owns 16-byte columns: it loads a column's sources for every accepted depth, then stores.
__global__ void __launch_bounds__(256) tree_compact_kernel(const DCompactArgs a) {
    __shared__ int s_tab[kTreeWords];
    griddep_wait();
    for (int i = threadIdx.x; i < kTreeWords; i += 256) s_tab[i] = a.table[i];
    __syncthreads();
    const int b = blockIdx.x, n_kv = a.n_swa + a.n_full;
    const bool cap = b >= n_kv;
    const int row_q = (cap ? a.cap_row_bytes : a.kv_row_bytes) / 16;  // 16-byte chunks a row
    const int q = cap ? (row_q + kCompactCapCtas - 1) / kCompactCapCtas : row_q;
    const int q0 = cap ? (b - n_kv) % kCompactCapCtas * q : 0, q1 = min(row_q, q0 + q);
    const int* slot = s_tab + (b < a.n_swa ? kTreeSlotSwa : kTreeSlotFull);
    uint4* buf = (uint4*)a.rows[cap ? n_kv + (b - n_kv) / kCompactCapCtas : b];
    const int acc = s_tab[kTreePath];
    for (int k = q0 + threadIdx.x; k < q1; k += 256) {
        uint4 v[kTreeRows - 1];
#pragma unroll
        for (int i = 1; i < kTreeRows; ++i)
            if (i <= acc && s_tab[kTreePath + i] != i) {
                const int r = s_tab[kTreePath + i];
                v[i - 1] = buf[(size_t)(cap ? r : slot[r]) * row_q + k];
            }
#pragma unroll
        for (int i = 1; i < kTreeRows; ++i)
            if (i <= acc && s_tab[kTreePath + i] != i) buf[(size_t)(cap ? i : slot[i]) * row_q + k] = v[i - 1];
    }
}

static cudaError_t launch_t(void (*kern)(DTreeArgs), dim3 grid, dim3 block, cudaStream_t s, bool pdl, const DTreeArgs& a) {
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

cudaError_t dtree_walk_launch(const DTreeArgs& a, cudaStream_t s, bool pdl) {
    return launch_t(dtree_walk_kernel, dim3(1), dim3(32), s, pdl, a);
}

cudaError_t tree_compact_launch(const DCompactArgs& a, cudaStream_t s, bool pdl) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.n_swa + a.n_full + kCompactCapCtas * a.n_cap);
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, tree_compact_kernel, a);
}

}  // namespace mk
