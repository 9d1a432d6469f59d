// Argument records and host entry points of the layer's kernels (one record per kernel, frozen at bind time).
#pragma once

#include "params.h"

namespace mk {

struct AttnArgs {
    const bf16* qkv;
    const unsigned char* k_cache;
    const unsigned char* v_cache;
    const long long* page_table;
    const int* kv_len;
    float* ws;
    bf16* x_attn;
    int M, qh, kvh, G, R, qkv_row, window, splits;
    const int* tree;  // a token-tree window's table (draft.h kTree*: depth at [16 + row], ancestor mask at [32 + row]) or null
};
struct NormArgs {
    int mode, H, ranks;
    const bf16* src;
    bf16* branch;
    const float* stream_in;
    const float* alpha;
    const float* beta;
    const bf16* pre_w;
    const bf16* post_w;
    float* stream_out;
    bf16* normed;
    float* normed_f32;
    int M;
    XchgWait wait;
};
struct TopkArgs {
    const float* logits;
    const float* bias;
    int* ids;
    float* w;
    double mult;
    float route_scale;
    int E, k, M;
    int* status;  // a row with NaN scores is recorded here (code 6); may be null
    const float* score;  // [M, E] selection scores from the router GEMM's epilogue, or null: computed here from the logits
    int e_lo, e_hi;      // e_hi > e_lo: the route tables keep the experts in [e_lo, e_hi) only (expert parallelism)
};
struct NqArgs {
    const bf16* pooled;
    const bf16* gamma;
    unsigned char* q;
    unsigned char* sf;
    float* x_scale;
    float eps;
    int P, bf16_out;
    XchgWait wait;
};
struct CombineArgs {
    const bf16* zb;
    const float* w;
    const bf16* gamma_p1;
    bf16* y;
    int P, k, b_live;
    XchgWait wait;
};
struct RowopsArgs {
    bf16* qkv;
    const float* cos_sin;
    const int* cache_loc;
    unsigned char* k_cache;
    unsigned char* v_cache;
    float q_scale, eps;
    int M, qh, kvh, qkv_row, kv_row_bytes;
};
struct ExpertArgs {
    const RouteTables* rt;
    int P, I, I_s, H_s, rank, ranks, topk, wbf16;
    const unsigned char* xq;
    const unsigned char* x_sf;
    const float* x_scale;
    const unsigned char* w1_gate;
    const unsigned char* w1_gate_sf;
    const unsigned char* w1_up;
    const unsigned char* w1_up_sf;
    const float* g1_alphas;
    const float* g1_scale_c;
    unsigned char* z_peer[kMaxRanks];
    unsigned char* zsf_peer[kMaxRanks];
    signed char* zex_peer[kMaxRanks];
    int n_peer;
    const unsigned char* z;
    const unsigned char* z_sfd;
    const float* rowscale;
    const unsigned char* w2;
    const unsigned char* w2_sf;
    const float* g2_alphas;
    bf16* zb_peer[kMaxRanks];
    XchgSignal sig_g1, sig_g2;  // the h planes (g1) and the expert outputs (g2) that go to every rank
    XchgWait wait_g2;           // a bf16 layer has no h-row kernel: g2 itself waits for the h planes
};

// gemm.cu: cluster split-K, no global scratch. gemm_plan fills wn / ksplit of a GEMM (-1: the shape has no valid plan).
int gemm_plan(bool wf32, int mode, int N, int K, int max_ctas, int* wn_out, int* ksplit_out);
size_t gemm_smem(const GemmArgs& a, bool wf32);
int gemm_grid(const GemmArgs& a);
cudaError_t gemm_prepare();
cudaError_t gemm_launch(const GemmArgs& a, bool wf32, cudaStream_t stream, bool pdl);

// gemm_gws.cu: split-K through global scratch (the stand-alone qkv head).
struct GemmGwsArgs {
    const void* w;        // [N, K] row-major weights (bf16 or f32)
    const void* x;        // [M, K] row-major activations (bf16, or f32 for f32 weights)
    int M, N, K;
    int ldw, ldx;         // row strides in elements
    float* partial;       // [ksplit, 16, N] f32 partial sums (ksplit > 1)
    unsigned* counter;    // [N / BN] arrival counters (zero between launches)
    void* out[kMaxRanks]; // destinations, each [M, ldo]
    int n_out;
    int ldo;              // row stride of out in elements
    int col0;             // first output column of this N range
    int out_f32;          // 1: f32 outputs, 0: bf16
};
int gemm_gws_ksplit(bool wf32, int K);
int gemm_gws_bn(bool wf32);
size_t gemm_gws_smem(bool wf32, int K, int ksplit);
cudaError_t gemm_gws_prepare();
cudaError_t gemm_gws_launch(const GemmGwsArgs& a, bool wf32, int ksplit, cudaStream_t stream, bool pdl);
cudaError_t attn_split_launch(const AttnArgs& a, cudaStream_t stream, bool pdl);
cudaError_t attn_combine_launch(const AttnArgs& a, cudaStream_t stream, bool pdl);
cudaError_t resid_norm_launch(const NormArgs& a, cudaStream_t s, bool pdl);
// one launch: block 0 routes (top-k + route tables), blocks 1..M run the pre-expert norm + quantisation of one row each
// `ticket`: a device word, zero between launches (the routing rows' arrivals)
cudaError_t route_nq_launch(const TopkArgs& t, const NqArgs& n, RouteTables* rt, int b_live, unsigned* ticket, cudaStream_t s, bool pdl);
cudaError_t hrow_launch(const unsigned char* z_sf, const signed char* z_ex, int groups, int slots_live, int slots,
                        unsigned char* z_sfd, float* rowscale, const XchgWait& wait, cudaStream_t s, bool pdl);
cudaError_t combine_launch(const CombineArgs& a, int M, cudaStream_t s, bool pdl);
cudaError_t rowops_launch(const RowopsArgs& a, cudaStream_t s, bool pdl);
size_t g1_smem(int P);
size_t g2_smem(int I);
cudaError_t experts_prepare();
cudaError_t g1_launch(const ExpertArgs& a, int max_active, cudaStream_t s, bool pdl);
cudaError_t g2_launch(const ExpertArgs& a, int max_active, cudaStream_t s, bool pdl);

// The tensor-core expert kernels (experts_umma.cu): one record per phase (g1 or g2).
struct UmmaArgs {
    const RouteTables* rt;
    int K;   // contraction length: P for g1, I for g2 (multiple of 256, at most 4096)
    int NB;  // 128-row blocks per expert: I_s / 128 (g1) or H_s / 128 (g2)
    int P, I, I_s, H_s, rank, topk;
    const unsigned char* wpack;  // [E][NB][K / 256][stage bytes] packed weight image
    const unsigned char* bq;     // B rows: g1 xq [M, P/2]; g2 z [slots, I/2]
    const unsigned char* bsf;    // their e4m3 scales: g1 x_sf [M, P/16]; g2 z_sfd [slots, I/16], or with `bex` the raw z_sf
    const signed char* bex;      // g2: the h planes' group exponents z_ex [slots, I/16]: the stager then forms the row view
                                 // itself (row exponent = the largest of the slot's exponents, every scale byte moved to it,
                                 // row scale 2^e_row) and no h-row kernel runs; null: bsf / rowscale hold the view
    XchgWait wait;               // g2 with bex: the h planes of every rank
    const float* x_scale;        // g1
    const float* g1_alphas;
    const float* g1_scale_c;
    const float* rowscale;       // g2: 2^e_row per slot
    const float* g2_alphas;
    unsigned char* z_peer[kMaxRanks];
    unsigned char* zsf_peer[kMaxRanks];
    signed char* zex_peer[kMaxRanks];
    bf16* zb_peer[kMaxRanks];
    int n_peer;
    int* status;
    XchgSignal sig;  // the exchange this phase's peer stores feed
};
// headtail.cu: the kernels around the decoder layers
struct FeedsArgs {
    const long long* positions;       // i64 [rows]
    const float* cos_sin_cache;       // f32 [cos_sin_rows, head_dim]
    long long cos_sin_rows;
    const long long* out_cache_loc;   // i64 [rows]
    const long long* swa_out_cache_loc;
    const long long* seq_lens;        // i64 [1]
    const long long* req_pool_indices;
    const int* req_to_token;          // i32 [r2t_rows, r2t_width]
    long long r2t_rows, r2t_width;
    const long long* full_to_swa;     // i64 [swa_map_len] or null
    long long swa_map_len;
    float* cos_sin;                   // out f32 [rows, head_dim]
    int* loc_full;
    int* loc_swa;
    int* kv_len;
    long long* pt_full;               // out i64 [r2t_width] byte offsets
    long long* pt_swa;
    int rows, head_dim, kv_row_bytes;
    int* status;
};
struct EntryArgs {
    const long long* ids;             // i64 [rows]
    const bf16* embed[kMaxRanks];     // every rank's vocab shard [shard_rows, hidden]
    long long shard_rows;
    int ranks;
    const bf16* pre_w;
    float* residual;                  // out f32 [rows, hidden]
    bf16* normed;                     // out bf16 [rows, hidden]
    int rows, hidden;
    float eps_embed, eps_pre;
};
struct SoftcapArgs {
    const float* x;
    float* out;
    long long numel;
    float scale, cap;
    XchgWait wait;
};
struct AcceptArgs {
    const float* logits;              // f32 [rows, vocab] gathered, before the soft cap
    int vocab, rows, b_live;
    float scale, cap;
    const long long* tokens;          // i64 [rows] the window's ids [anchor, d_1 ..]
    const int* accept_override;       // forced accepts per iteration (mod n_override) or null
    int n_override;
    long long* words;                 // i64 [8]: P, ANCHOR, ACCEPT, COMMIT, ITER, OUT_COUNT
    int* out_ring;
    int ring;
    int* top1;                        // out i32 [rows]
    unsigned* counter;                // one arrival counter, zero between launches
    const float* cos_sin_cache;       // f32 [cos_sin_rows, 64]
    long long cos_sin_rows;
    float* cos_sin;                   // next target feeds (any may be null)
    int* loc_full;
    int* loc_swa;
    int* kv_len;
    const float* dcos_sin_cache;      // f32 [dcos_sin_rows, 128]
    long long dcos_sin_rows;
    float* dcos_sin;                  // next draft feeds: [2 B, 128]
    int* dslot;
    int* dkv_len;
    int dring;
    XchgWait wait;                    // the lm_head shards of every rank
    long long pool_rows;              // 0: unchecked
    int* status;
    // the sampled accept (samp non-null) instead of the greedy one
    const long long* samp;            // i64 [4]: seed, stream, top_k, f32 temperature bits | f32 top_p bits << 32
    const long long* cand;            // i64 [b_live - 1][16] the draft slots' candidates
    const float* walk_q;              // f32 [b_live - 1][16] the walk's probabilities over them
    int block_verify;                 // 1: block verification, 0: token by token
    float* ys;                        // scratch f32 [rows][vocab]: soft-capped logits / T
    double* es;                       // scratch f64 [rows][vocab]: exp(y - max) of the kept entries, 0 elsewhere
    double* row_z;                    // scratch f64 [rows]: the kept mass
    double* sample_out;               // out f64 [2] or null: the residual's scale and the bonus distribution's mass
    int* tree;                        // the token tree's table (draft.h kTree*), or null: the window is a chain
};
cudaError_t feeds_launch(const FeedsArgs& a, cudaStream_t s, bool pdl);
cudaError_t entry_launch(const EntryArgs& a, cudaStream_t s, bool pdl);
cudaError_t softcap_launch(const SoftcapArgs& a, cudaStream_t s, bool pdl);
cudaError_t accept_launch(const AcceptArgs& a, cudaStream_t s, bool pdl);
cudaError_t headtail_prepare();

// segments.cuh (compiled with rows.cu): the dense GEMMs and the row work between them as two persistent kernels
struct SegGemm {
    const unsigned char* w;  // [N, K] row-major
    const unsigned char* x;  // [M, K] row-major (bf16, or f32 with f32 weights)
    long long ldw, ldx;      // row strides in bytes
    int N, K, M;
    int f32;                 // 1: f32 weights through tf32 (tile 16 rows), 0: bf16 (tile 64 rows)
    float* part;             // [K / 256][16][N] f32 partial sums (a slot per K chunk; few of them are written, see segments.cuh)
    int item0, per;          // set on the device: the GEMM's first item within its stage, items per CTA
    int packed;              // 1: w holds item images [N block][K chunk][rows][512 k + 64 bytes] (a few bulk copies per item);
                             // 2: w holds the tensor-core tile images of dense.cu ([tile][K stage][2 atoms][128 rows][128 B],
                             // 128-byte swizzle) and the GEMM runs on tcgen05 (dense_umma_kernel)
    // dense.cu only: stream-K partial sums [tiles][maxc][16][128] f32 live in `part`; one self-resetting ticket per tile
    int maxc;                // partial-sum slots per tile (an upper bound of the CTAs that share a tile's K range)
    unsigned* ticket;        // [tiles], zero between launches
};
struct GridBarrier {
    unsigned long long* count;  // starts at a multiple of the grid size and only grows
    long long budget;
    int* status;
};
struct SegAArgs {  // o_proj .. routing
    SegGemm oproj, pooler, router;
    bf16* ar_out[kMaxRanks];    // every present rank's all-reduce workspace
    int n_ar;
    long long ar_off;           // this rank's slot in a workspace (elements)
    XchgSignal sig_ar;
    NormArgs post_norm;
    bf16* pool_out[kMaxRanks];  // the node group's gather rows
    int n_pool, pool_ld, pool_col0;
    XchgSignal sig_pool;
    float* logits;
    TopkArgs topk;
    NqArgs nq;
    RouteTables* rt;
    int b_live;
    GridBarrier gb;
    int* status;
};
struct SegBArgs {  // combine .. successor's qkv head
    CombineArgs combine;
    int M;
    SegGemm unpool, qkv;
    bf16* unpool_out[kMaxRanks];
    int n_unpool, unpool_ld, unpool_col0;
    XchgSignal sig_unpool;
    NormArgs cross_norm;
    GemmArgs qkv_epi;           // the epilogue operands of the qkv head (out, cos_sin, cache_loc, pools, scales)
    int tail;                   // 1: no successor (the cross-layer norm is the final norm)
    GridBarrier gb;
    int* status;
};
// The DFlash2 draft's row work that rides the finishes of its GEMMs (draft.h holds the rest of the draft's records).
struct DQkvRowsArgs {
    const bf16* qkv;  // [M][(qh + 2 kvh) x 128]
    int M, qh, kvh;
    const bf16* q_norm;
    const bf16* k_norm;
    float eps;
    const float* rope;  // [rope_rows][128]: cos | sin
    long long rope_rows;
    const long long* words;
    bf16* q_out;        // [M][qh x 128]
    bf16* k_pool;       // [pool_rows][kvh][128], slot = position % pool_rows
    bf16* v_pool;
    long long pool_rows;
    int* status;
};

struct SegConv {  // the grouped conv's side 0 over the rows the projection was computed from
    const bf16* h;     // [M][H]
    const bf16* base;  // [2 sides][2 taps][H]
    bf16* xa;          // [M][H]
    int H, groups;
};
struct SegGemmArgs {  // one GEMM stage (or pooler + router) as a kernel of its own
    SegGemm g[2];
    int n_gemm;
    int finish;                 // 0: bf16 push of g[0]; 1: the same plus f32 logits and routing scores of g[1]; 2: qkv row ops;
                                // 3: SwiGLU of g[0]'s [gate | up] columns; 4: f32 push of g[0] (out holds float pointers);
                                // 5: conv projection + conv; 6: the draft's qkv + row work
    bf16* out[kMaxRanks];
    int n_out;
    long long ldo, off0;
    XchgSignal sig;
    float* f32_out;
    float* score;
    const float* score_bias;
    double score_mult;
    GemmArgs epi;               // finish 2: the qkv head's epilogue operands
    SegConv conv;               // finish 5: g[0] is a conv projection; bf16 coefficients to out[0], then the conv's side 0
    DQkvRowsArgs rows;          // finish 6: g[0] is the draft's qkv; bf16 rows to out[0], head norm, neox RoPE, K / V append
    GridBarrier gb;
    int* status;
};
// Launches the GEMM stage on the engine its weights are packed for (g[0].packed == 2: dense.cu's tcgen05 kernel).
cudaError_t seg_gemm_launch(const SegGemmArgs& a, int grid, cudaStream_t s, bool pdl);
size_t segments_smem();
// dense.cu: the tcgen05 stream-K GEMM kernel over tile images (SegGemm.packed == 2)
size_t dense_smem();
cudaError_t dense_prepare();
int dense_grid(const SegGemmArgs& a, int sms);
size_t dense_part_bound(long long N);  // floats of partial-sum scratch that any K and any grid leave sufficient for N rows
// `force_grid` > 0: the kernel that runs the stage has that many CTAs (a fused kernel: one grid for all its stages)
bool dense_setup(SegGemmArgs& a, int sms, float* part, size_t part_floats, unsigned* ticket, size_t ticket_words, int force_grid = 0);
cudaError_t dense_launch(const SegGemmArgs& a, int sms, cudaStream_t s, bool pdl);
cudaError_t segments_prepare();
cudaError_t seg_a_launch(const SegAArgs& a, int grid, cudaStream_t s, bool pdl);
cudaError_t seg_b_launch(const SegBArgs& a, int grid, cudaStream_t s, bool pdl);

// fused.cuh (compiled with rows.cu): two GEMM stages on the tensor-core engine and the row work around them in one kernel
struct FusedArgs {
    SegGemmArgs st[2];          // the GEMM stages (tile images, dense_setup done with the kernel's grid)
    int n_stages;               // 1 or 2
    int row_kind[3];            // the row stage before stage 0 / between the stages / behind the last: 0 none, 1 norm rows,
                                // 2 routing + pre-expert norm and quantisation rows, 3 combine rows
    int M;                      // window rows
    NormArgs norm;
    TopkArgs topk;
    float* score_out;           // [M, E] the routing's selection scores (topk.score reads them), written by the top-k CTAs
    NqArgs nq;
    RouteTables* rt;
    int b_live;
    CombineArgs combine;
    // words of this kernel in the layer's private scratch (zero once, they only grow)
    unsigned* launches;         // launches completed
    unsigned* done;             // CTAs out of the current launch
    unsigned* dep;              // [6]: parts of row stage 0 / 1 done, router tiles finished, first-GEMM tiles of stage 0 / 1 finished,
                                // top-k rows done
    int norm_parts, combine_parts;  // 1024-column parts a norm row (H / 1024) / a combine row (ceil(P / 1024)) is cut into
    float* meet_part;           // partial sums of the rows' parts: 2 norm meetings x [16 rows][8 parts], then the combine's
                                // [16 rows][4 parts][8 slots]
    unsigned* meet_count;       // [3][16] arrivals per row of the three meetings, only grow
    int tiles0[2];              // tiles of each stage's first GEMM
    int router_tiles;
    int router_contribs;        // CTAs that hold a K range of a router tile, over all its tiles (each arrives once per launch)
    // exchanges fed per finished tile: stage 0's first GEMM (sig0), stage 1's first GEMM (sig1); flag words of the fused
    // protocol in every receiving rank's flag block
    XchgSignal sig0, sig1;
    const unsigned* wait_flag[2];   // this rank's word of the exchange stage s feeds (null: no exchange)
    const unsigned* wait_epoch[2];  // the flag block's count of completed launches that fed it
    unsigned wait_contrib[2];       // arrivals per launch: present ranks x tiles
    int wait_stage[2];              // recorded with a wait that ran out
    unsigned* bump_epoch[2];        // the counts the last CTA out advances (null: none)
    long long budget;
    int* status;
};
size_t fused_smem();
cudaError_t fused_prepare();
cudaError_t fused_launch(const FusedArgs& a, int grid, cudaStream_t s, bool pdl);

size_t experts_umma_smem(bool g2);
// experts_bf16_umma.cu: the bf16 experts as a grouped GEMM on the tcgen05 dense pipeline (tile images per expert)
struct Bf16UmmaArgs {
    const RouteTables* rt;
    const unsigned char* w;  // [E][NB][K bytes / 256][32768] tile images (g1: [gate | up] rows in silu_perm order)
    const bf16* x;           // g1: the normed pooled rows [M, K] (row = slot / topk); g2: the gathered h rows [slots, K]
    int K;                   // contraction length in elements (a multiple of 128)
    int NB;                  // 128-row tiles per expert: 2 I_s / 128 (g1) or H_s / 128 (g2)
    int topk, by_token, g2;
    bf16* out[kMaxRanks];    // g1: every rank's h rows [slots, ldo], g2: every rank's expert outputs [slots, ldo]
    int n_out;
    long long ldo, col0;     // this rank's column band starts at col0; a tile covers 64 (g1) or 128 (g2) columns of it
    float* part;             // [2 x grid][16][128] f32: the accumulators of the unit pieces a CTA shares with its neighbours
    unsigned* ticket;        // [grid] arrivals at a shared unit, zero between launches
    XchgWait wait;           // g2: the h rows of every rank
    XchgSignal sig;
    int* status;
};
size_t experts_bf16_umma_smem();
cudaError_t experts_bf16_umma_prepare();
cudaError_t experts_bf16_umma_launch(const Bf16UmmaArgs& a, int grid, cudaStream_t s, bool pdl);
constexpr int kBf16UmmaMaxGrid = 160;
constexpr size_t kBf16UmmaScratchBytes = (size_t)2 * kBf16UmmaMaxGrid * 2048 * 4 + 2 * kBf16UmmaMaxGrid * 4;  // pieces, then g1's and g2's tickets

cudaError_t experts_umma_prepare();
cudaError_t experts_umma_launch(const UmmaArgs& a, bool g2, int grid, cudaStream_t s, bool pdl);


}  // namespace mk
