// Argument records and launchers of the DFlash2 draft's row kernels (draft.cu). The draft's GEMMs run on the item engine
// (seg_gemm_launch); everything between them is here: feature rows, norms with the all-reduce and the conv finish folded
// in, the grouped conv, the qkv row work (head norm, neox RoPE, K/V append), the non-causal window attention, the
// candidate top-k, the selector lattice and walk, the pool sync.
#pragma once

#include "stages.h"

namespace mk {

constexpr int kDraftHeadDim = 128;
constexpr int kDraftTopK = 16;
constexpr int kDraftMaxLayers = 8;
constexpr int kDraftKeysPerSplit = 64;
constexpr int kDraftTopkChunk = 4096;  // vocabulary entries one top-k CTA scans
constexpr int kMaxMergeChunks = 128;    // chunk lists the merge holds in registers (256 threads x 8 keys)
// step words (i64): the draft reads the position, the anchor and the last commit
constexpr int kWordP = 0, kWordAnchor = 1, kWordCommit = 3, kWordIter = 4;
// exchange points of the draft's own flag block
enum DraftXchg { DXP_CTX = 0, DXP_ATTN, DXP_MLP, DXP_LOGITS = 5 };

struct DFeatsArgs {
    const float* cap[8];  // captured residuals, f32 [rows][hidden] each
    int n_cap;
    bf16* feats;          // [rows][n_cap x hidden]
    int rows, hidden;
};

// h = rms_norm(x [+ residual]) x w, residual' = bf16(x + residual). The row source x is one of: plain bf16 rows; the sum
// (rank order, f32, rounded to bf16) of the ranks' partials in an all-reduce workspace, finished by the conv's side 1;
// the block's embedding rows [anchor, mask, mask, ...].
struct DNormArgs {
    const bf16* x;         // plain rows [M][H], or null
    const bf16* ar;        // [ranks][16][H] partials, or null
    int ranks;
    const bf16* coeff;     // [M][2 x 2 x groups] conv projection of the sublayer input (side 1 is read)
    const bf16* base;      // [2 sides][2 taps][H]
    int groups;
    const long long* words;   // embedding source: the anchor's word
    const bf16* embed[8];     // every rank's vocab shard
    long long shard_rows;
    int emb_ranks;            // > 0: the embedding source
    long long mask_id;
    const bf16* residual;  // [M][H] or null (the source is then its own residual)
    const bf16* w;         // [H]
    bf16* h;               // [M][H]
    bf16* res_out;         // [M][H] or null
    bf16* x_out;           // the source rows as consumed ([M][H], for checks) or null
    int M, H;
    float eps;
    XchgWait wait;
    int* status;
};

struct DConvArgs {  // side 0: out[n] = (b0 + d[n][0]) h[n] + (b1 + d[n][1]) h[n - 1]
    const bf16* h;
    const bf16* coeff;
    const bf16* base;
    bf16* out;
    int M, H, groups;
};

struct DCtxKvArgs {
    const bf16* kv;  // [M][layers x 2 x kvh x 128]: per layer the k heads, then the v heads
    int M, layers, kvh;
    const bf16* k_norm[kDraftMaxLayers];
    bf16* k_pool[kDraftMaxLayers];
    bf16* v_pool[kDraftMaxLayers];
    long long pool_rows;
    float eps;
    const float* rope;
    long long rope_rows;
    const long long* words;
    int* status;
};

struct DAttnArgs {
    const bf16* q;  // [M][qh x 128]
    const bf16* k_pool;
    const bf16* v_pool;
    long long pool_rows;
    const long long* words;
    float* ws;      // [kvh][nsplit][M x G][132]: m, l, two pad words, O (16-byte aligned)
    bf16* o;        // [M][qh x 128]
    int M, qh, kvh, left, nsplit;
};

struct DTopkArgs {
    const float* logits;  // [gamma][V] f32 (rounded to bf16 before the comparison)
    long long V;
    int gamma, nchunk;
    unsigned long long* keys;  // [gamma][nchunk + 1][16]: the chunks' lists, then the row's merged 16
    unsigned* row_count;       // [gamma] arrival counters of the rows' chunk CTAs (self-resetting)
    XchgWait wait;
};

struct DLatticeArgs {
    const unsigned long long* keys;
    int gamma, nchunk;
    const bf16* hid;  // [gamma][R]
    int R;
    const bf16* pred;  // [V][R]
    const bf16* succ;
    long long vocab;
    const long long* words;
    float mult, cap;
    long long* cand;     // [gamma][16]
    float* unary;        // [gamma][16]
    float* scores;       // [gamma][16][16]
    int* pick;           // [gamma]
    long long* drafts;   // [gamma]
    long long* verify_ids;  // [gamma + 1]: the anchor, then the drafts
    unsigned* counter;
    int* status;
    // the sampled walk (temperature > 0), or samp null: the greedy walk
    const long long* samp;  // i64 [4]: seed, stream, top_k, f32 temperature bits | f32 top_p bits << 32
    float* walk_q;          // [gamma][16]: each slot's probabilities over its candidates
};

struct DKvSyncArgs {
    const long long* words;
    const long long* window;  // [16] this iteration's window slots
    long long* state;         // [17]: the position the pool is complete to, then the saved window slots
    const unsigned long long* ring;  // [n_buf] base pointers
    const unsigned long long* pool;
    int n_buf, row_bytes;
    long long ring_rows;
    int lag;
    int* status;
};

// tree.cu: the token tree. The table's words (i32): parent, depth, ancestor mask, accepted path ([0] the accept length,
// [i] the window row at depth i), the window rows' slots in the full and the sliding-window pools.
constexpr int kTreeRows = 16;
constexpr int kTreeParent = 0, kTreeDepth = 16, kTreeMask = 32, kTreePath = 48, kTreeSlotFull = 64, kTreeSlotSwa = 80, kTreeWords = 96;
constexpr int kCompactCapCtas = 4;
struct DTreeArgs {
    const long long* cand;   // [rows - 1][16]
    const float* scores;     // [rows - 1][16][16]
    const long long* words;  // the anchor
    int* table;              // out [kTreeWords]
    long long* verify_ids;   // out [rows]: the rows' tokens in preorder
    const int* loc_full;     // [rows] the window rows' pool slots (or null)
    const int* loc_swa;
    int rows;
    const float* cos_sin_cache;  // f32 [cos_sin_rows][64] or null
    long long cos_sin_rows;
    float* cos_sin;              // out [rows][64]: the target's rotation rows, row r at position P + depth(r)
};
struct DCompactArgs {
    const int* table;                 // the path and the window's slots
    const unsigned long long* rows;   // [n_swa + n_full + n_cap] base pointers: sliding-window pools, full pools, capture buffers
    int n_swa, n_full, n_cap;
    int kv_row_bytes, cap_row_bytes;  // multiples of 16
};

// One kernel of a draft launch record (the host walks an array of these).
enum DraftOpKind {
    DOP_FEATS = 1, DOP_GEMM, DOP_NORM, DOP_CONV, DOP_QKV_ROWS, DOP_CTX_KV, DOP_ATTN_SPLIT, DOP_ATTN_MERGE, DOP_TOPK, DOP_LATTICE,
    DOP_KV_SYNC, DOP_TREE, DOP_COMPACT
};
struct DraftOp {
    int kind;
    union {
        DFeatsArgs feats;
        SegGemmArgs gemm;
        DNormArgs norm;
        DConvArgs conv;
        DQkvRowsArgs rows;
        DCtxKvArgs ckv;
        DAttnArgs attn;
        DTopkArgs topk;
        DLatticeArgs lat;
        DKvSyncArgs sync;
        DTreeArgs tree;
        DCompactArgs compact;
    };
};

cudaError_t dfeats_launch(const DFeatsArgs& a, cudaStream_t s, bool pdl);
cudaError_t dnorm_launch(const DNormArgs& a, cudaStream_t s, bool pdl);
cudaError_t dconv_launch(const DConvArgs& a, cudaStream_t s, bool pdl);
cudaError_t dqkv_rows_launch(const DQkvRowsArgs& a, cudaStream_t s, bool pdl);
cudaError_t dctx_kv_launch(const DCtxKvArgs& a, cudaStream_t s, bool pdl);
cudaError_t dattn_split_launch(const DAttnArgs& a, cudaStream_t s, bool pdl);
cudaError_t dattn_merge_launch(const DAttnArgs& a, cudaStream_t s, bool pdl);
cudaError_t dtopk_launch(const DTopkArgs& a, cudaStream_t s, bool pdl);
cudaError_t dlattice_launch(const DLatticeArgs& a, cudaStream_t s, bool pdl);
cudaError_t dkv_sync_launch(const DKvSyncArgs& a, cudaStream_t s, bool pdl);
cudaError_t dtree_walk_launch(const DTreeArgs& a, cudaStream_t s, bool pdl);
cudaError_t tree_compact_launch(const DCompactArgs& a, cudaStream_t s, bool pdl);
cudaError_t draft_prepare();
size_t dattn_smem();

}  // namespace mk
