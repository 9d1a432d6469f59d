// C ABI of the B200 (sm_100a) decode-layer library, libmk_b200.so.
//
// Conventions are those of the reference's host ABI (sgl_muse_mega/muse_spark/sm103/host/abi.h:1-9): every bind struct
// holds only uint64_t / int64_t / double fields, one declaration per line (device pointers as uint64_t, 0 = absent);
// every int-returning function returns 0 on success and -1 on failure with the reason in mk_last_error(); the caller
// owns all device memory, the library owns the MkModule / MkLaunch handles; a launch is bound ONCE and
// mk_launch(handle, stream, pdl) is the only per-step call (no allocation, no synchronisation: graph-capturable).
//
// Differences from the reference, by design: the kernels are linked into the library (no cubin file is loaded, so
// mk_module_load takes image == NULL), shapes are run-time fields of MkLayerShape instead of per-image compile-time
// constants, and device-side waits never trap: they give up after a bound and record why in a status block that
// mk_launch_status reads.
#pragma once

#include <stdint.h>

// capacity of the peer arrays: the largest tensor-parallel world (abi.h:15)
#define MKH_RANKS 8
// stages of one layer launch, in launch order (mk_launch_step runs a sub-range)
#define MKH_LAYER_STAGES 17

#ifdef __cplusplus
extern "C" {
#endif

typedef struct MkModule MkModule;
typedef struct MkLaunch MkLaunch;

// replaces abi.h:24 mk_last_error
const char* mk_last_error(void);

// replaces abi.h:30 mk_module_load. The kernels are built into this library: image must be NULL and bytes 0. Binds the
// module to the calling thread's current CUDA device, which must be compute capability 10.x.
int mk_module_load(const void* image, uint64_t bytes, const char* code_prefetch_prefix, MkModule** out);
// replaces abi.h:36 mk_module_free
void mk_module_free(MkModule* module);

// replaces abi.h:40 mk_launch. Enqueues every kernel of the bound launch on `stream` (a cudaStream_t as an integer);
// pdl != 0 adds the programmatic-dependent-launch attribute to every kernel, the first included (it then overlaps
// its prologue with the tail of whatever kernel precedes it on the stream, e.g. the previous layer's last kernel).
int mk_launch(const MkLaunch* launch, uint64_t stream, int pdl);
// Test hook with no counterpart in the reference: enqueues stages [first, first + count) only. Lets a test interleave
// the stages of several ranks' launches on one GPU, so that their exchanges run without the ranks waiting on each other.
int mk_launch_step(const MkLaunch* launch, uint64_t stream, int64_t first, int64_t count);
// replaces abi.h:41 mk_launch_free
void mk_launch_free(MkLaunch* launch);

// replaces abi.h:43-51 MkLaunchInfo / mk_launch_info
typedef struct MkLaunchInfo {
    int64_t grid;         // largest grid among the launch's kernels
    int64_t block;        // largest block
    int64_t cluster;      // cluster width (1: none)
    int64_t smem;         // largest dynamic shared memory request
    int64_t kernels;      // kernels enqueued by one mk_launch
    int64_t param_bytes;  // bytes of the packed parameter record
} MkLaunchInfo;
int mk_launch_info(const MkLaunch* launch, MkLaunchInfo* out);

// Stands where abi.h:53 mk_launch_params stands (the reference's launch is one kernel whose parameter block that call
// copies out; here a launch is a list of kernels with one argument record each). Renders, for a layer launch, what the bind
// wired between those kernels as text, one `name key=value ...` line per producer and consumer of an exchange point:
//   post_norm wait=packets present=0x3 band=0 contributors=0     (wait: off | counter | packets)
//   o_proj signal=0 remote=0 target=0                            (signal: receivers' flag words; 0 = none)
// Works on pack-only records (bound without a module), for tests that check a bind on the CPU. Returns the text's length
// (without the terminator), -1 when `cap_bytes` is too small or the launch is not a layer launch.
int mk_launch_params(const MkLaunch* launch, char* text, uint64_t cap_bytes);

// No counterpart in the reference (its waits trap, K/README.md:111-121). Copies the launch's device status block to the
// host (synchronises the stream first). code 0 = clean; otherwise the wait that gave up.
typedef struct MkLaunchStatus {
    int64_t code;      // 0 ok, 1 an exchange wait ran out (a peer never signalled), 3 a bulk copy or tensor-core barrier
                       // never completed, 4 an out-of-range position / request index was clamped, 6 a row's router
                       // scores were NaN (it is routed to the lowest expert ids; its outputs are meaningless)
    int64_t stage;     // stage index that recorded it (exchange waits), or a kernel-specific site number
    int64_t block;     // blockIdx.x
    int64_t observed;  // value seen
    int64_t expected;  // value waited for
} MkLaunchStatus;
int mk_launch_status(const MkLaunch* launch, uint64_t stream, MkLaunchStatus* out);

// ---- one decoder layer ----

// Run-time shape of one rank's layer launch (the reference bakes these per image: abi.h:60-101 MkLayerConstants).
typedef struct MkLayerShape {
    int64_t rows;         // window rows M (1..16)
    int64_t hidden;       // model width H
    int64_t moe_hidden;   // expert width P (pooler output)
    int64_t q_heads;      // this rank's query heads
    int64_t kv_heads;     // this rank's kv heads
    int64_t experts;      // routed experts E
    int64_t topk;         // experts per row
    int64_t inter;        // full expert intermediate I
    int64_t ranks;        // tensor-parallel world
    int64_t node_ranks;   // ranks of a node group (pooler / unpooler gathers)
    int64_t rank;         // this rank
    int64_t window;       // sliding window (keys p with pos - p <= window); 0 = global attention
    int64_t bf16;         // 1: bf16 experts, 0: NVFP4
    int64_t tail;         // 1: last layer (ends at the final norm, no successor head)
    int64_t next_rope;    // 1: the successor is a sliding-window layer (RoPE rows applied)
} MkLayerShape;

// Buffer extents the caller allocates for a shape (replaces abi.h:60-102 mk_layer_constants).
typedef struct MkLayerConstants {
    int64_t stages;          // kernels per launch
    int64_t slots;           // route slots = rows x topk
    int64_t qkv_row;         // [q | k | v | o-gate] row width
    int64_t kv_row_bytes;    // one K (or V) pool row
    int64_t inter_rank;      // I / ranks
    int64_t hidden_rank;     // P / ranks (W2 rows per rank)
    int64_t ar_bytes;        // all-reduce workspace: ranks x rows x H bf16
    int64_t pool_ag_bytes;   // pooler gather row block: rows x P bf16
    int64_t unpool_ag_bytes; // unpooler gather: rows x H bf16
    int64_t z_bytes;         // gathered h codes: slots x I/2 (bf16 variant: slots x I x 2)
    int64_t z_sf_bytes;      // gathered h scales: slots x I/16
    int64_t z_ex_bytes;      // gathered h exponents: slots x I/16 (int8)
    int64_t zb_bytes;        // gathered expert outputs: slots x P bf16
    int64_t ws_bytes;        // private scratch (attention partials, split-K partials, counters, route tables)
    int64_t attn_splits;     // split-KV partitions per kv head
    int64_t flag_words;      // u32 exchange flags per rank
    int64_t status_bytes;    // device status block
} MkLayerConstants;
int mk_layer_constants(const MkLayerShape* shape, MkLayerConstants* out);

// One layer launch's operands (replaces abi.h:106-211 MkLayerBind; same names where the meaning is the same).
typedef struct MkLayerBind {
    // attention
    uint64_t qkv_in;      // this layer's head row [rows, qkv_row] bf16 (written by the predecessor)
    uint64_t k_cache;     // this layer's pool, [kv_rows, kv heads x 64] bf16
    uint64_t v_cache;
    int64_t kv_rows;
    uint64_t page_table;  // i64 [page_stride] byte offsets by position
    uint64_t kv_len;      // i32 [1]: context length + rows
    int64_t page_stride;
    uint64_t x_attn;      // out [rows, q_heads x 64] bf16
    // o_proj + all-reduce + post-attention norm
    uint64_t w_o;         // [H, q_heads x 64] bf16
    uint64_t ar;          // this rank's all-reduce workspace (ar_bytes)
    uint64_t ar_peer[MKH_RANKS];  // every rank's workspace (own included); 0 = rank absent (slot pre-filled)
    uint64_t branch;      // out [rows, H] bf16 (the all-reduce sum)
    uint64_t stream_in;   // [rows, H] f32
    uint64_t alpha;
    uint64_t beta;
    uint64_t prenorm_w;
    uint64_t stream_out;  // out [rows, H] f32 (the post-attention residual)
    uint64_t h3;          // out [rows, H] bf16
    uint64_t h3f;         // out [rows, H] f32
    // pooler || router -> top-k -> pre-expert norm + quant -> route tables
    uint64_t w_p;         // [P, H] bf16 (replicated; this rank computes its node block)
    uint64_t pool_ag;     // this rank's pooler gather buffer
    uint64_t pool_ag_peer[MKH_RANKS];
    uint64_t w_r;         // [E, H] f32
    uint64_t logits;      // out [rows, E] f32
    double router_mult;
    uint64_t expert_bias;
    uint64_t topk_idx32;  // out [rows, topk] i32
    uint64_t topk_w;      // out [rows, topk] f32
    double route_scale;
    uint64_t gamma;       // pre-expert norm weight [P] bf16
    double eps;
    uint64_t q;           // out: NVFP4 rows [rows, P/2] u8 (bf16 variant: [rows, P] bf16)
    uint64_t sf;          // out [rows, P/16] u8
    uint64_t x_scale;     // out [rows] f32
    // experts
    uint64_t w1_gate;     // NVFP4: [E, I_s, P/2] u8; bf16: [E, I_s, P] bf16
    uint64_t w1_gate_sf;  // [E, I_s, P/16] u8
    uint64_t w1_up;
    uint64_t w1_up_sf;
    uint64_t w2;          // NVFP4: [E, H_s, I/2] u8; bf16: [E, H_s, I] bf16
    uint64_t w2_sf;       // [E, H_s, I/16] u8
    uint64_t w1_pack;     // NVFP4 tensor-core image of W1, [E, I_s/128, P/256, 36864] u8 (weights.pack_w1_fp4); 0 = absent
    uint64_t w2_pack;     // image of W2, [E, H_s/128, I/256, 18432] u8 (weights.pack_w2_fp4). With both images bound the
                          // experts run on tcgen05 and the plain w1_* / w2* tensors may be 0; without, on CUDA cores
    uint64_t g1_alphas;
    uint64_t g1_scale_c;
    uint64_t g2_alphas;
    uint64_t z;           // gathered h planes of this rank
    uint64_t z_sf;
    uint64_t z_ex;
    uint64_t zb;
    uint64_t z_peer[MKH_RANKS];
    uint64_t zsf_peer[MKH_RANKS];
    uint64_t zex_peer[MKH_RANKS];
    uint64_t zb_peer[MKH_RANKS];
    uint64_t gamma_p1;
    uint64_t y;           // out [rows, P] bf16
    // next-layer phase
    uint64_t w_up;        // unpooler [H, P] bf16
    uint64_t unpool_ag;
    uint64_t unpool_ag_peer[MKH_RANKS];
    uint64_t c_alpha;
    uint64_t c_beta;
    uint64_t c_pre_w;
    uint64_t c_post_w;
    uint64_t c_stream_out;  // out [rows, H] f32
    uint64_t h3q;           // out [rows, H] bf16: the successor's normed input (tail: the final norm's rows)
    uint64_t w_qkv;         // successor's [qkv_row, H] bf16
    uint64_t qkv_out;       // out [rows, qkv_row] bf16
    uint64_t cos_sin;       // [rows, 64] f32
    uint64_t cache_loc;     // i32 [rows]: pool slots of the window's rows
    uint64_t next_k_cache;
    uint64_t next_v_cache;
    int64_t next_kv_rows;
    double q_scale;
    double qkv_eps;
    // exchange flags and private scratch
    // The flag block: u32 [flag_words], zeroed once by the caller, one per rank; it may be shared by all launches of a
    // rank (the layers of a stack, the lm_head, the accept). Words [0, 8): one counter per exchange point (0 all-reduce,
    // 1 pooler gather, 2 h planes, 3 expert outputs, 4 unpooler gather, 5 logits), advanced by every contributing rank's
    // producer kernel once per launch; words [8, 24) are the owner's bookkeeping. flags 0: no signalling, the launches of
    // the ranks are ordered by the caller (all ranks on one stream).
    uint64_t flags;
    uint64_t flags_peer[MKH_RANKS];  // the peers' flag blocks (0: absent), same presence as the *_peer data buffers
    uint64_t ws;            // ws_bytes of private scratch, zeroed once by the caller
    uint64_t status;        // status_bytes, zeroed once by the caller
    int64_t b_live;         // live window rows (abi.h:208-210)
    int64_t wait_budget;    // polls before an exchange wait gives up (0: library default)
    // Form of the dense stages (o_proj, pooler, router, unpooler, successor's qkv head), for shapes whose K dimensions are
    // multiples of 512 (others always get form 2):
    //   0  one launch per stage, the GEMMs on a persistent item engine (one 512-thread CTA per SM streams 64-row x 512-k
    //      items through two buffers, partial sums per K chunk, one grid barrier, then the epilogue); pooler and router share
    //      a launch: 13 kernels a layer;
    //   1  mk_launch runs o_proj .. routing and combine .. qkv head as two persistent kernels with grid barriers between their
    //      stages: 7 kernels a layer. Their exchange waits poll for peers that run at the same time: for a lone rank or one
    //      process per GPU, never for several ranks launched one after the other on one GPU; mk_launch_step still runs
    //      form 0;
    //   2  one launch per stage with the cluster split-K GEMMs: 14 kernels a layer.
    // mk_launch_info.kernels tells which form was bound.
    int64_t fused;
    // 1: w_o, w_p, w_r, w_up and w_qkv are item images of the item engine instead of row-major matrices (forms 0 and 1
    // only): [ceil(N / 64)][K / 512][64 rows][512 k + 32 pad] bf16 ([N / 16][K / 512][16 rows][512 k + 16 pad] f32 for
    // w_r), rows past N zero; w_p and w_up then hold this rank's node block only (P / node_ranks and H / node_ranks
    // rows). One bulk copy brings an item in, instead of one per weight row.
    int64_t dense_packed;
    // Expert parallelism of the expert block (whole experts per rank instead of the reference's tensor-parallel slices):
    // with expert_hi > expert_lo this launch's route tables keep only the routed (row, slot) pairs whose expert id lies
    // in [expert_lo, expert_hi), so g1, g2 and their zb rows cover this rank's experts alone; the other pairs' zb rows
    // are the other ranks' to write (into the same zb buffer) before combine reads them. The expert arrays are still
    // indexed by the global id: a rank that holds only its experts passes base pointers moved back by expert_lo experts.
    // 0 / 0: every expert (the reference's layout).
    int64_t expert_lo;
    int64_t expert_hi;
    // An expert-parallel world of one process per GPU (ep_world > 1, with an expert range on a ranks = 1 shape and the packed
    // NVFP4 images): this launch is rank ep_rank of ep_world; g2 stores its zb rows into every rank's zb (zb_peer[r], r <
    // ep_world; zb_peer[ep_rank] may be 0 = zb) and signals the expert-output exchange in every rank's flag block
    // (flags_peer[r]); combine waits for all ep_world ranks. 0 / 0: no such world (the ranks of an expert-parallel world
    // emulated on one GPU share zb and run one after the other).
    int64_t ep_rank;
    int64_t ep_world;
    // A token-tree window (0: a chain): the table mk_dflash_tree_bind's launch writes (i32 [96]). The attention then places
    // row r at position context + depth[r] and lets it see, of the window's own rows, the rows of its ancestor mask (every
    // context key is its past); the K / V rows are still appended at the window's slots in row order (the compaction moves
    // the accepted path's rows afterwards), and cos_sin must hold the rows' rotations by depth (the tree's launch writes them).
    uint64_t tree;
    // 1: the four bf16 exchanges of the layer (all-reduce partials, pooler gather, expert outputs, unpooler gather) carry
    // their own validity instead of counting in the flag block: ar, pool_ag, zb and unpool_ag of every rank must be filled
    // with 0xFF bytes once before the first launch (a bf16 of all ones marks "not arrived"; no kernel produces it). The
    // producers then only store (no fence, no arrival, no flag), the consumers poll the 16-byte packets they use with the
    // wait budget and put the mark back, so the buffers read as marks after a step: a caller that inspects ar / pool_ag /
    // zb / unpool_ag between stages binds 0. With tile images (dense_packed 2) the router's f32 logits are handed to the
    // routing rows the same way (fill logits with 0xFF bytes as well; they read as marks afterwards), and the row kernels
    // that consume packets do not wait for the producing grid's end. The reference's counterpart: its packets with in-band validity
    // (kernels/postattn.cuh:38-53, kernels/framework.cuh:1409-1482). Not with fused = 1. 0: counter words (flags) or, without
    // a flag block, stream order.
    int64_t packets;
} MkLayerBind;
int mk_layer_bind(MkModule* module, const MkLayerShape* shape, const MkLayerBind* bind, MkLaunch** out);

// ---- the rest of the verify step ----

// Window feeds (replaces abi.h:216-239 MkFeedsBind / mk_feeds_bind, same field names): the step's RoPE rows, cache-write
// slots, kv_len and the position -> byte-offset tables of one request.
typedef struct MkFeedsBind {
    uint64_t positions;          // i64 [rows]
    uint64_t cos_sin_cache;      // f32 [cos_sin_rows, head_dim]; 0 = the rope rows are written elsewhere
    int64_t cos_sin_rows;
    uint64_t out_cache_loc;      // i64 [rows]
    uint64_t swa_out_cache_loc;  // i64 [rows] or 0
    uint64_t seq_lens;           // i64 [1]
    uint64_t req_pool_indices;   // i64 [1]
    uint64_t req_to_token;       // i32 [r2t_rows, r2t_width]
    int64_t r2t_rows;
    int64_t r2t_width;
    uint64_t full_to_swa;        // i64 [swa_map_len] or 0
    int64_t swa_map_len;
    uint64_t cos_sin;            // out f32 [rows, head_dim]
    uint64_t loc_full;           // out i32 [rows]
    uint64_t loc_swa;            // out i32 [rows]
    uint64_t kv_len;             // out i32 [1]
    uint64_t pt_full;            // out i64 [r2t_width]
    uint64_t pt_swa;             // out i64 [r2t_width] or 0
    int64_t rows;
    int64_t head_dim;
    int64_t kv_row_bytes;
    uint64_t status;             // i32 [16] or 0: an out-of-range position or request index is recorded here (code 4), not trapped
} MkFeedsBind;
int mk_feeds_bind(MkModule* module, const MkFeedsBind* bind, MkLaunch** out);

// The fused entry (replaces abi.h:242-254 MkEntryBind / mk_entry_bind): embedding row from the owning rank's vocab
// shard, weightless embed norm, layer 0's pre-attention norm.
typedef struct MkEntryBind {
    uint64_t ids;                    // i64 [rows]
    uint64_t embed_peer[MKH_RANKS];  // every rank's vocab shard [shard_rows, hidden] bf16
    int64_t shard_rows;
    int64_t ranks;
    uint64_t pre_w;                  // bf16 [hidden]
    uint64_t residual;               // out f32 [rows, hidden]
    uint64_t normed;                 // out bf16 [rows, hidden]
    int64_t rows;
    int64_t hidden;
    double eps_embed;
    double eps_pre;
} MkEntryBind;
int mk_entry_bind(MkModule* module, const MkEntryBind* bind, MkLaunch** out);

// lm_head (replaces abi.h:257-270 MkLmHeadBind / mk_lm_head_bind): this rank's vocab shard against the final hidden
// rows, f32, written into every present rank's gathered logits row at column col0 (peer stores; the reference multicasts).
typedef struct MkLmHeadBind {
    uint64_t w;                    // bf16 [n_out, hidden]: the rank's vocab rows
    uint64_t x;                    // bf16 [rows, hidden]
    uint64_t out_peer[MKH_RANKS];  // every rank's gathered logits f32 [rows, v_total] (own included); 0 = absent
    int64_t rank;
    int64_t v_total;
    int64_t col0;
    int64_t n_out;
    int64_t hidden;
    int64_t rows;
    uint64_t status;               // i32 [16] or 0: a weight copy that never landed is recorded here (code 3), not trapped
    uint64_t flags;                // this rank's flag block and the peers' (as MkLayerBind); 0: no signalling
    uint64_t flags_peer[MKH_RANKS];
    uint64_t ws;                   // 0, or ws_bytes of private scratch zeroed once: with hidden a multiple of 512 the GEMM then
    int64_t ws_bytes;              // runs on the item engine (needs (hidden / 256) x 16 x n_out x 4 + 512 bytes)
    int64_t w_packed;              // 1: w holds item images (as MkLayerBind.dense_packed; needs ws)
} MkLmHeadBind;
int mk_lm_head_bind(MkModule* module, const MkLmHeadBind* bind, MkLaunch** out);

// Soft cap over the gathered logits (replaces abi.h:273-286 MkSoftcapBind / mk_softcap_bind).
typedef struct MkSoftcapBind {
    uint64_t x;    // f32 [numel]
    uint64_t out;  // f32 [numel]
    int64_t numel;
    double scale;
    double cap;
    uint64_t flags;        // this rank's flag block: wait for `contributors` lm_head shards per launch; 0: no wait
    int64_t contributors;
    int64_t wait_budget;   // polls (0: library default)
    uint64_t status;       // i32 [16] or 0: a wait that ran out is recorded here (code 1)
} MkSoftcapBind;
int mk_softcap_bind(MkModule* module, const MkSoftcapBind* bind, MkLaunch** out);

// Greedy verify-accept on the gathered logits (replaces the accept half of abi.h mk_dflash_verify_accept_bind; the
// lm_head half is mk_lm_head_bind): first-arg-max of the soft-capped rows, greedy prefix accept or the forced table,
// the step words [P, ANCHOR, ACCEPT, COMMIT, ITER, OUT_COUNT, -, -], the committed-token ring, the next step's feeds.
typedef struct MkAcceptBind {
    uint64_t logits;           // f32 [rows, vocab] gathered, before the soft cap
    int64_t vocab;
    int64_t rows;
    int64_t b_live;
    double scale;
    double cap;
    uint64_t tokens;           // i64 [rows]: the window's ids [anchor, d_1 ..]
    uint64_t accept_override;  // i32 [n_override] forced accept per iteration, or 0
    int64_t n_override;
    uint64_t words;            // i64 [8], read and advanced
    uint64_t out_ring;         // i32 [ring]
    int64_t ring;
    uint64_t top1;             // out i32 [rows]
    uint64_t counter;          // u32 [512], zeroed once by the caller (arrival counters and the row chunks' winners)
    uint64_t cos_sin_cache;    // f32 [cos_sin_rows, 64]
    int64_t cos_sin_rows;
    uint64_t cos_sin;          // out: next target feeds (each may be 0)
    uint64_t loc_full;
    uint64_t loc_swa;
    uint64_t kv_len;
    uint64_t dcos_sin_cache;   // f32 [dcos_sin_rows, 128]
    int64_t dcos_sin_rows;
    uint64_t dcos_sin;         // out: next draft feeds [2 b_live, 128] (each may be 0)
    uint64_t dslot;
    uint64_t dkv_len;
    int64_t dring;
    uint64_t flags;            // as MkSoftcapBind
    int64_t contributors;
    int64_t wait_budget;
    uint64_t status;
    int64_t pool_rows;         // rows of the KV pools behind loc_full / loc_swa (identity slots): a next window that would
                               // not fit is clamped to the last rows and recorded (code 4); 0 = unchecked
    // The sampled accept (reference kernels/dflash/sample.cuh sample_accept; arithmetic test/reference/dflash2.py:703-791)
    // instead of the greedy one when samp is bound: the rows' sampling distributions (temperature, exact top-k and top-p
    // sets), block verification (block_verify 1) or the token-by-token test against the draft walk's probabilities, the
    // bonus token from the residual by inverse CDF in vocabulary order. Same launch, same outputs (top1 is not written).
    uint64_t samp;             // i64 [4] as MkDflashDraftHeadBind.samp (seed, stream, top_k, temperature | top_p bits), or 0
    uint64_t cand;             // i64 [b_live - 1, 16]: the draft slots' candidates (MkDflashDraftHeadBind.cand)
    uint64_t walk_q;           // f32 [b_live - 1, 16]: the walk's probabilities over them (MkDflashDraftHeadBind.walk_q)
    int64_t block_verify;
    uint64_t sample_ws;        // scratch of sample_ws_bytes >= rows x vocab x 12 + 256, 256-byte aligned
    int64_t sample_ws_bytes;
    uint64_t sample_out;       // out f64 [16] or 0: [0] the residual's scale, [1] the mass of the bonus distribution
                               // (the rest is written by trace builds only)
    // The token tree (greedy accept only): the table mk_dflash_tree_bind's launch wrote (i32 [96]), or 0 for a chain. The
    // accept then takes the deepest row whose token and all of whose ancestors' tokens equal the target's arg-max at their
    // parents (accept_override names the leaf row instead), commits the path's tokens and the bonus, and writes the path
    // into the table ([48] the accept length, [48 + i] the window row at depth i) for mk_dflash_tree_compact_bind.
    uint64_t tree;
} MkAcceptBind;
int mk_accept_bind(MkModule* module, const MkAcceptBind* bind, MkLaunch** out);

// ---- memory shared between the ranks' processes ----

// Replaces the reference's symmetric allocations (sm103/buffers.py Symmetric, made there through torch's symmetric-memory
// rendezvous): one process per GPU allocates its exchange buffers once, hands the 64-byte handle to its peers through any
// channel (the host side uses torch.distributed.all_gather_object), and every peer maps the allocation into its own
// address space; the kernels then store into the peers' buffers directly over NVLink. Plain CUDA IPC handles: no
// multicast object is ever bound to the memory.
#define MK_SYMM_HANDLE_BYTES 64
int mk_symm_alloc(int64_t bytes, uint64_t* ptr, unsigned char* handle);  // device memory on the current device, zeroed
int mk_symm_open(const unsigned char* handle, uint64_t* ptr);            // a peer's allocation, peer access enabled on demand
int mk_symm_close(uint64_t ptr);                                         // unmaps what mk_symm_open returned
int mk_symm_free(uint64_t ptr);                                          // frees what mk_symm_alloc returned

// ---- layer 0's head: qkv GEMM + qk-norm + RoPE + K/V append as a stand-alone launch ----

// Replaces abi.h:255-270 MkQkvBind / mk_qkv_bind (same names for the same operands); rows, heads and the scratch are
// run-time fields here.
typedef struct MkQkvBind {
    uint64_t w;          // [qkv_row, hidden] bf16, rows [q | k | v | o-gate]
    uint64_t x;          // [rows, hidden] bf16 normed input
    uint64_t out;        // [rows, qkv_row] bf16
    uint64_t cos_sin;    // [rows, 64] f32 {cos[32] | sin[32]}; 0 = no RoPE (global layer)
    uint64_t cache_loc;  // i32 [rows] pool slots of the window's rows
    uint64_t k_cache;    // [kv_rows, kv_heads x 64] bf16; 0 = no append
    uint64_t v_cache;
    double q_scale;
    double eps;
    int64_t hidden;
    int64_t rows;
    int64_t q_heads;
    int64_t kv_heads;
    uint64_t ws;         // ws_bytes of scratch (split-K partial sums and arrival counters), zeroed once by the caller
    int64_t ws_bytes;
} MkQkvBind;
typedef struct MkQkvConstants {
    int64_t qkv_row;       // 2 (q_heads + kv_heads) 64
    int64_t kv_row_bytes;  // kv_heads x 64 bf16
    int64_t ws_bytes;      // scratch the bind needs
    int64_t kernels;       // kernels per launch
} MkQkvConstants;
int mk_qkv_constants(const MkQkvBind* bind, MkQkvConstants* out);
int mk_qkv_bind(MkModule* module, const MkQkvBind* bind, MkLaunch** out);

// No counterpart in the reference. The same head (qkv GEMM + qk norm + RoPE + K/V append) for callers that must not
// allocate: a serving process whose memory pool claimed the whole device at start-up, so that a later cudaMalloc fails or
// fragments it, or a latency-critical section where an allocation would stall the device. Nothing is allocated, on the
// device or through any library: the split-K partial sums and arrival counters live in a fixed 4 MiB + 4 KiB array that is
// part of the library's device image (every GPU that loads the library holds it until the process exits). `ws` and
// `ws_bytes` of the bind are ignored; every other field means what it means for mk_qkv_bind, and no MkLaunch is created:
// the call enqueues the kernels on `stream` directly.
// Limits: qkv_row = 2 (q_heads + kv_heads) 64 <= 4096 and hidden <= 8192; larger shapes are refused with an error.
// The first call on a device looks up the array's address for that device (the device must be current) and should
// therefore be made before any stream capture begins. All calls share the one array: two calls whose kernels overlap on
// the GPU (different streams, no dependency) race on it; calls on one stream are safe back to back.
int mk_qkv_launch_static(const MkQkvBind* bind, uint64_t stream);

// ---- DFlash2 draft --------------------------------------------------------------------------------------------------------
// The draft's half of a fused decode iteration (reference abi.h:301-545, :645-660; kernels/dflash/{head,layer,kv_sync}.cu):
// context update, the block forward through the draft's layers, the candidate head with the selector lattice and walk, the
// pool sync. Unlike the reference's per-image binds (one .so per kernel, weights in tile-packed layouts) the binds here
// take the plain row-major shards and each yields a launch record of several kernels; every GEMM runs on the item engine
// (64 rows x 512 k items), the row work between them in small kernels. Head dimension 128, 2 conv taps, top-16.
//
// The draft has a flag block of its own (as MkLayerBind.flags: 32 u32, zeroed once): exchange points 0 = gathered fc rows,
// 1 / 2 = the attention / MLP sublayer's all-reduce, 5 = the draft's gathered logits.
// Step words (i64): [0] P, the anchor's position; [1] the anchor token; [3] the last commit length.
typedef struct MkDflashShape {
    int64_t rows;          // block B (1 anchor + B - 1 mask rows), <= 16
    int64_t hidden;        // multiple of 512, <= 8192
    int64_t layers;        // <= 8
    int64_t q_heads;       // this rank's
    int64_t kv_heads;      // this rank's
    int64_t inter;         // this rank's MLP columns, multiple of 512
    int64_t features;      // captured target layers (fc K = features x hidden), <= 8
    int64_t ranks;
    int64_t rank;
    int64_t window_left;   // keys a query sees on each side
    int64_t conv_groups;   // hidden / conv group size
    int64_t vocab;         // whole vocabulary
    int64_t selector_rank; // even, <= 512
} MkDflashShape;
typedef struct MkDflashConstants {
    int64_t ws_bytes;      // private scratch every draft bind of this shape shares (GEMM partial sums, barrier word, walk counter)
    int64_t attn_splits;   // 64-key blocks the attention cuts the window into
    int64_t attn_ws_bytes; // attention partials
    int64_t topk_chunks;   // candidate lists per row
    int64_t coeffs;        // conv coefficients per row: 2 sides x 2 taps x groups
    int64_t qkv_row;       // (q_heads + 2 kv_heads) x 128
    int64_t kv_rows_n;     // layers x 2 x kv_heads x 128: the context update's k / v columns
} MkDflashConstants;
int mk_dflash_constants(const MkDflashShape* shape, MkDflashConstants* out);

// draft entry (reference mk_dflash_entry_bind, abi.h:322-349): feats = bf16(cap), ctx_raw = feats fc^T gathered over the
// ranks, ctx = rms(ctx_raw) x hid_norm, every layer's context K (head norm, RoPE) / V rows of the last commit into the
// draft's pools, then the block's embedding rows [anchor, mask ...] and layer 0's input norm. 6 kernels.
typedef struct MkDflashEntryBind {
    uint64_t cap[8];        // f32 [rows][hidden] each: the last verify's captured residuals
    uint64_t words;
    uint64_t embed_peer[8]; // every rank's vocab shard of the target embedding, bf16 [shard_rows][hidden]
    int64_t shard_rows;
    int64_t mask_id;
    uint64_t w_fc;          // bf16 [hidden / ranks][features x hidden]
    uint64_t hid_norm;
    uint64_t in_norm;       // layer 0's input norm
    uint64_t w_kv;          // bf16 [kv_rows_n][hidden]: per layer its k rows, then its v rows
    uint64_t k_norm[8];
    uint64_t k_pool[8];     // bf16 [pool_rows][kv_heads][128] per layer, slot = position % pool_rows
    uint64_t v_pool[8];
    int64_t pool_rows;
    uint64_t rope;          // f32 [rope_rows][128]: cos | sin by position
    int64_t rope_rows;
    uint64_t feats;         // bf16 [rows][features x hidden]
    uint64_t ctx_raw_peer[8];  // bf16 [rows][hidden] on every present rank (own included)
    uint64_t ctx;           // bf16 [rows][hidden]
    uint64_t kv;            // bf16 [rows][kv_rows_n]
    uint64_t x;             // bf16 [rows][hidden]: the block's embedding rows = layer 0's residual
    uint64_t h;             // bf16 [rows][hidden]: layer 0's normed input
    uint64_t ws;
    uint64_t flags;
    uint64_t flags_peer[8];
    uint64_t status;
    int64_t wait_budget;
    double eps;
    int64_t packed;         // 1: w_fc and w_kv are item images (as MkLayerBind.dense_packed)
} MkDflashEntryBind;
int mk_dflash_entry_bind(MkModule* module, const MkDflashShape* shape, const MkDflashEntryBind* bind, MkLaunch** out);

// one draft layer from its normed input (reference mk_dflash_qkv_bind + mk_dflash_layer_bind, abi.h:353-491): conv
// projection, conv, qkv, head norm + RoPE + K/V append, attention, o_proj partial pushed to every rank, all-reduce + conv
// finish + post norm, conv projection, conv, gate_up with SwiGLU, down partial pushed, all-reduce + conv finish + the
// successor's norm (the next layer's input norm, or the final norm). 10 kernels: the conv rides its projection's finish, the
// head norm + RoPE + K/V append the qkv GEMM's.
typedef struct MkDflashLayerBind {
    uint64_t h_in;          // bf16 [rows][hidden]
    uint64_t res_in;
    uint64_t words;
    uint64_t attn_proj;
    uint64_t attn_base;  // bf16 [coeffs][hidden], [2][2][hidden]
    uint64_t mlp_proj;
    uint64_t mlp_base;
    uint64_t w_qkv;         // bf16 [qkv_row][hidden]: q rows, k rows, v rows
    uint64_t q_norm;
    uint64_t k_norm;
    uint64_t w_o;           // bf16 [hidden][q_heads x 128]
    uint64_t post_norm;
    uint64_t w_gate_up;     // bf16 [2 inter][hidden]: gate rows, then up rows
    uint64_t w_down;        // bf16 [hidden][inter]
    uint64_t next_norm;     // the successor's norm weight
    uint64_t k_pool;
    uint64_t v_pool;
    int64_t pool_rows;
    uint64_t rope;
    int64_t rope_rows;
    uint64_t c_att;
    uint64_t xa;
    uint64_t qkv;
    uint64_t q;
    uint64_t attn_ws;
    uint64_t o;   // bf16 [rows][coeffs], [rows][hidden], [rows][qkv_row], [rows][q x 128], f32 partials, bf16 [rows][q x 128]
    uint64_t ar_attn_peer[8];                  // bf16 [ranks][16][hidden] on every present rank
    uint64_t a;             // bf16 [rows][hidden] or 0: the finished attention sublayer output (for checks)
    uint64_t h_post;
    uint64_t res_post;
    uint64_t c_mlp;
    uint64_t xm;
    uint64_t m;  // bf16 [rows][coeffs], [rows][hidden], [rows][inter]
    uint64_t ar_mlp_peer[8];
    uint64_t x_out;         // bf16 [rows][hidden] or 0: the finished MLP sublayer output (for checks)
    uint64_t h_out;         // bf16 [rows][hidden]: the successor's normed input (the draft's y after the last layer)
    uint64_t res_out;       // bf16 [rows][hidden], or 0 after the last layer
    uint64_t ws;
    uint64_t flags;
    uint64_t flags_peer[8];
    uint64_t status;
    int64_t wait_budget;
    double eps;
    int64_t packed;         // 1: attn_proj, mlp_proj, w_qkv, w_o, w_gate_up, w_down are item images
} MkDflashLayerBind;
int mk_dflash_layer_bind(MkModule* module, const MkDflashShape* shape, const MkDflashLayerBind* bind, MkLaunch** out);

// draft head after the draft's own lm_head launch (mk_lm_head_bind over y rows 1.., f32 logits gathered on every rank;
// reference mk_dflash_draft_head_bind, abi.h:497-544): hid = y W_P^T, per-row top-16 of the bf16-rounded logits (ties to
// the smaller id), soft cap, the lattice score[e][p][c] = unary[e][c] + bf16(<bf16(A[pred] hid[e]), S[cand[e][c]]>), the
// greedy walk, the verify window's ids. 3 kernels.
typedef struct MkDflashDraftHeadBind {
    uint64_t y;             // bf16 [rows][hidden]; rows 1 .. are read
    uint64_t w_hproj;       // bf16 [selector_rank][hidden]
    uint64_t hid;           // bf16 [rows - 1][selector_rank]
    uint64_t logits;        // f32 [rows - 1][vocab]
    uint64_t pred_codebook;
    uint64_t succ_codebook;  // bf16 [vocab][selector_rank]
    uint64_t words;
    uint64_t keys;          // u64 [rows - 1][topk_chunks + 1][16]: the chunks' candidate lists, then the row's merged 16
    uint64_t cand;          // i64 [rows - 1][16]
    uint64_t unary;         // f32 [rows - 1][16]
    uint64_t scores;        // f32 [rows - 1][16][16]
    uint64_t pick;          // i32 [rows - 1]
    uint64_t drafts;        // i64 [rows - 1]
    uint64_t verify_ids;    // i64 [rows]: the anchor, then the drafts
    double mult;
    double cap;
    uint64_t ws;
    uint64_t flags;         // the logits exchange is awaited when given
    int64_t contributors;
    uint64_t status;
    int64_t wait_budget;
    int64_t packed;         // 1: w_hproj is an item image
    // the sampled walk (reference abi.h:537-540, kernels/dflash/sample.cuh walk): samp = i64 [4] sampling words (seed,
    // stream, top_k, f32 temperature bits | f32 top_p bits << 32) or 0 for the greedy walk; slot e then draws its candidate
    // from softmax(score row / T) with the Philox4x32-10 uniform e of {words[4] (iteration), stream, purpose 0}
    uint64_t samp;
    uint64_t walk_q;        // f32 [rows - 1][16] or 0: each slot's probabilities over its candidates
} MkDflashDraftHeadBind;
int mk_dflash_draft_head_bind(MkModule* module, const MkDflashShape* shape, const MkDflashDraftHeadBind* bind, MkLaunch** out);

// draft_kv_sync (reference abi.h:645-660, kernels/dflash/kv_sync.cu): the committed positions' K / V rows from the draft's
// pools into the serving engine's draft pool at the slots it allocated. state i64 [17]: the position the pool is complete
// to, then the slots of the next positions. A pool and ring that disagree by more than 16 rows copy nothing and record
// status code 4 (the reference traps).
// The token tree (reference kernels/dflash/tree.cuh). mk_dflash_tree_bind: the draft head's tree walk, after its lattice:
// the window's 16 rows as a tree over the candidates (best-first by path log-probability, four successors a row, preorder),
// table i32 [96] = parent[16] (-1 for the anchor), depth[16], ancestor mask[16], path[16] (the accept's), the window rows'
// slots in the full and the sliding-window pools (copied from loc_full / loc_swa when given); verify_ids = the rows' tokens;
// cos_sin = the target's rotation feeds of the window rewritten by depth.
typedef struct MkDflashTreeBind {
    uint64_t cand;        // i64 [rows - 1][16]
    uint64_t scores;      // f32 [rows - 1][16][16]
    uint64_t words;       // the step words (the anchor)
    uint64_t table;       // out i32 [96]
    uint64_t verify_ids;  // out i64 [rows]
    uint64_t loc_full;    // i32 [rows] or 0
    uint64_t loc_swa;     // i32 [rows] or 0
    int64_t rows;         // 16
    uint64_t cos_sin_cache;  // f32 [cos_sin_rows][64] or 0
    int64_t cos_sin_rows;
    uint64_t cos_sin;        // out f32 [rows][64] or 0: the target's rotation rows of the window, row r at P + depth(r)
} MkDflashTreeBind;
int mk_dflash_tree_bind(MkModule* module, const MkDflashTreeBind* bind, MkLaunch** out);

// mk_dflash_tree_compact_bind (reference abi.h mk_dflash_tree_compact, tree.cuh:251-298): after the tree accept, the row at
// depth i (1 .. accept) of every K / V pool and capture buffer takes the bytes of the accepted path's row. rows: a device
// array of base pointers, the sliding-window pools first (rows addressed through the table's sliding-window slots), then
// the full pools, then the capture buffers (rows addressed by window row).
typedef struct MkDflashTreeCompactBind {
    uint64_t table;
    uint64_t rows;          // u64 [n_swa + n_full + n_cap]
    int64_t n_swa;
    int64_t n_full;
    int64_t n_cap;
    int64_t kv_row_bytes;   // multiple of 16
    int64_t cap_row_bytes;  // multiple of 16
} MkDflashTreeCompactBind;
int mk_dflash_tree_compact_bind(MkModule* module, const MkDflashTreeCompactBind* bind, MkLaunch** out);

typedef struct MkDflashKvSyncBind {
    uint64_t words;
    uint64_t window;   // i64 [16]
    uint64_t state;    // i64 [17]
    uint64_t ring;     // u64 [n_buf] device array of base pointers
    uint64_t pool;     // u64 [n_buf]
    int64_t n_buf;
    int64_t row_bytes; // multiple of 16
    int64_t ring_rows;
    int64_t lag;
    uint64_t status;
} MkDflashKvSyncBind;
int mk_dflash_kv_sync_bind(MkModule* module, const MkDflashKvSyncBind* bind, MkLaunch** out);

#ifdef __cplusplus
}
#endif
