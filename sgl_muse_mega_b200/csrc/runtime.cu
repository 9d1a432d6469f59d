// Host side of the C ABI (include/mk_abi.h): module handle, bind-once launch records, the layer's launch list.
// Counterpart of the reference's host launcher (sm103/host/runtime.cu:429-520 core, :679-989 layer bind): bind checks
// every operand once and freezes one argument record per kernel; mk_launch only enqueues.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>

#include "../../include/mk_abi.h"
#include "draft.h"
#include "stages.h"

namespace mk {

// ---- errors ----
static thread_local char g_error[512] = "";

static int fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return -1;
}

#define MK_REQUIRE(cond, ...) \
    do {                      \
        if (!(cond)) return fail(__VA_ARGS__); \
    } while (0)

static int cuda_fail(cudaError_t e, const char* what) { return fail("%s: %s", what, cudaGetErrorString(e)); }

}  // namespace mk

struct MkModule {
    int device;
    int sms;  // streaming multiprocessors: the persistent kernels launch one CTA per SM
};

enum Stage {
    ST_ATTN_SPLIT = 0, ST_ATTN_COMBINE, ST_OPROJ, ST_POST_NORM, ST_POOLER, ST_ROUTER, ST_TOPK, ST_NQ, ST_TABLES, ST_G1,
    ST_HROW, ST_G2, ST_COMBINE, ST_UNPOOL, ST_CROSS_NORM, ST_QKV, ST_ROWOPS, ST_COUNT
};
static_assert(ST_COUNT == MKH_LAYER_STAGES, "stage list and ABI constant disagree");

struct MkLaunch {
    bool pack_only;
    int device;
    MkLayerShape shape;
    MkLayerConstants consts;
    MkLayerBind bind;
    mk::AttnArgs attn;
    mk::GemmArgs oproj, pooler, router, unpool, qkv;
    mk::GemmGwsArgs head_gemm;  // the stand-alone qkv head (split-K through global scratch)
    int head_ks;
    bool is_head;
    mk::NormArgs post_norm, cross_norm;
    mk::TopkArgs topk;
    mk::NqArgs nq;
    mk::CombineArgs combine;
    mk::RowopsArgs rowops;
    mk::ExpertArgs ex;
    mk::RouteTables* rt;
    unsigned* route_ticket;  // the routing rows' arrivals (route_nq_kernel)
    unsigned char* z_sfd;
    float* rowscale;
    int* status;
    int max_active, slots_live;
    bool use_umma;  // experts on tcgen05 (packed images bound) instead of CUDA cores
    int sms;
    mk::UmmaArgs umma_g1, umma_g2;
    mk::Bf16UmmaArgs bf16_g1, bf16_g2;
    bool use_bf16_umma;  // a bf16 layer's experts on tcgen05 (tile images bound)
    bool stage_on[ST_COUNT];
    mk::XchgWait hrow_wait;
    bool use_segments;  // mk_launch runs the dense stages as the two persistent segment kernels
    bool seg_gemms;     // the per-stage list runs its GEMMs on the item engine (pooler + router in one launch)
    mk::SegGemmArgs sg_oproj, sg_pool, sg_unpool, sg_qkv;
    mk::SegAArgs seg_a;
    mk::SegBArgs seg_b;
    bool use_fused;     // mk_launch runs the dense stages as the two fused tensor-core kernels (fused.cuh)
    mk::FusedArgs fused_a, fused_b;
    int fused_grid_a, fused_grid_b;
    // stand-alone launches around the layers (feeds, entry, lm_head, soft cap, accept): n_ops > 0 replaces the stage list
    int n_ops;
    int op_kind[4];
    mk::FeedsArgs feeds;
    mk::EntryArgs entry;
    mk::SoftcapArgs softcap;
    mk::AcceptArgs accept;
    mk::GemmArgs op_gemm;
    // the DFlash2 draft's launch lists: n_dops > 0 replaces both of the above
    mk::DraftOp* dops;
    int n_dops;
};
// exchange points (word index in a rank's flag block) and the default poll budget of a wait (a poll is one round trip to
// the L2, 0.5 - 1 us: seconds)
enum XchgPoint { XP_AR = 0, XP_POOL, XP_Z, XP_ZB, XP_UNPOOL, XP_LOGITS };
static const long long kDefaultWaitBudget = 1ll << 22;
enum OpKind { OP_FEEDS = 1, OP_ENTRY, OP_GEMM_BF16, OP_SOFTCAP, OP_ACCEPT };

using namespace mk;

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static int attn_splits_for(const MkLayerShape& s) {
    // Global attention: two 256-thread CTAs fit an SM (128 registers a thread), so 288 CTAs over the kv heads; at run time
    // only as many splits as the context has 64-key blocks take part (attention.cu attn_span). The merge holds up to 256.
    int sp = 288 / (int)s.kv_heads;
    if (sp < 1) sp = 1;
    if (sp > 256) sp = 256;
    // a sliding-window layer never sees more than window + rows keys
    if (s.window > 0) {
        const int blocks = (int)((s.window + s.rows + 63) / 64) + 1;
        if (sp > blocks) sp = blocks;
    }
    return sp;
}

static int check_shape(const MkLayerShape* s) {
    MK_REQUIRE(s != nullptr, "shape is NULL");
    MK_REQUIRE(s->rows >= 1 && s->rows <= kMaxRows, "rows %lld outside 1..16", (long long)s->rows);
    MK_REQUIRE(s->topk >= 1 && s->rows * s->topk <= kMaxSlots, "rows x topk %lld exceeds %d", (long long)(s->rows * s->topk), kMaxSlots);
    MK_REQUIRE(s->topk <= 32, "topk %lld exceeds 32", (long long)s->topk);
    MK_REQUIRE(s->experts >= s->topk && s->experts <= 1024 && s->experts % 16 == 0, "experts %lld unsupported", (long long)s->experts);
    MK_REQUIRE(s->ranks == 1 || s->ranks == 2 || s->ranks == 4 || s->ranks == 8, "ranks %lld not 1/2/4/8", (long long)s->ranks);
    MK_REQUIRE(s->rank >= 0 && s->rank < s->ranks, "rank %lld outside the world", (long long)s->rank);
    MK_REQUIRE(s->node_ranks >= 1 && s->ranks % s->node_ranks == 0, "node_ranks %lld does not divide ranks", (long long)s->node_ranks);
    MK_REQUIRE(s->hidden >= 256 && s->hidden <= 8192 && s->hidden % 256 == 0, "hidden %lld unsupported", (long long)s->hidden);
    MK_REQUIRE(s->moe_hidden % (32 * s->node_ranks) == 0 && s->moe_hidden % (16 * s->ranks) == 0 && s->moe_hidden % 256 == 0 &&
                   s->moe_hidden <= 4096,
               "moe_hidden %lld unsupported", (long long)s->moe_hidden);
    MK_REQUIRE(s->inter % (16 * s->ranks) == 0 && s->inter % 32 == 0 && s->inter <= 6144, "inter %lld unsupported", (long long)s->inter);
    MK_REQUIRE(s->hidden % (32 * s->node_ranks) == 0, "hidden %lld not divisible over the node group", (long long)s->hidden);
    MK_REQUIRE(s->q_heads >= 1 && s->kv_heads >= 1 && s->q_heads % s->kv_heads == 0, "heads %lld / %lld", (long long)s->q_heads, (long long)s->kv_heads);
    MK_REQUIRE(s->rows * (s->q_heads / s->kv_heads) <= 128, "rows x heads per kv head exceeds 128");
    MK_REQUIRE(s->window >= 0, "negative window");
    MK_REQUIRE(s->experts % 16 == 0 && s->hidden % 64 == 0, "experts / hidden are not whole GEMM tiles");
    return 0;
}

static void fill_constants(const MkLayerShape& s, MkLayerConstants* c) {
    memset(c, 0, sizeof *c);
    const int64_t M = s.rows, slots = s.rows * s.topk;
    c->stages = ST_COUNT;
    c->slots = slots;
    c->qkv_row = 2 * (s.q_heads + s.kv_heads) * kHeadDim;
    c->kv_row_bytes = s.kv_heads * kHeadDim * 2;
    c->inter_rank = s.inter / s.ranks;
    c->hidden_rank = s.moe_hidden / s.ranks;
    c->ar_bytes = s.ranks * M * s.hidden * 2;
    c->pool_ag_bytes = M * s.moe_hidden * 2;
    c->unpool_ag_bytes = M * s.hidden * 2;
    c->z_bytes = s.bf16 ? slots * s.inter * 2 : slots * s.inter / 2;
    c->z_sf_bytes = slots * s.inter / 16;
    c->z_ex_bytes = slots * s.inter / 16;
    c->zb_bytes = slots * s.moe_hidden * 2;
    c->attn_splits = attn_splits_for(s);
    c->flag_words = 64;
    c->status_bytes = 4096;
    // scratch carve: attention partials | gemm partials | gemm counters | route tables | z_sfd | rowscale
    const int64_t R = M * (s.q_heads / s.kv_heads);
    size_t off = 0;
    off += align_up((size_t)s.kv_heads * c->attn_splits * R * 66 * 4, 256);
    int64_t nmax = c->qkv_row;
    if (s.hidden > nmax) nmax = s.hidden;
    off += align_up((size_t)32 * 16 * nmax * 4, 256);  // up to 32 K chunks (256 k each) of [16, N] f32
    off += align_up((size_t)1024 * 4, 256);
    off += align_up(sizeof(RouteTables), 256);
    off += align_up((size_t)slots * s.inter / 16, 256);
    off += align_up((size_t)slots * 4, 256);
    if (s.bf16) off += align_up(kBf16UmmaScratchBytes, 256);  // the grouped tensor-core experts' pieces and tickets
    c->ws_bytes = (int64_t)off;
}

extern "C" {

const char* mk_last_error(void) { return g_error; }

int mk_module_load(const void* image, uint64_t bytes, const char* code_prefetch_prefix, MkModule** out) {
    (void)code_prefetch_prefix;
    MK_REQUIRE(out != nullptr, "out is NULL");
    MK_REQUIRE(image == nullptr && bytes == 0, "this library carries its kernels: pass image NULL, bytes 0");
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceProperties");
    MK_REQUIRE(prop.major == 10, "device %d is compute capability %d.%d; the kernels are built for sm_100a", dev, prop.major, prop.minor);
    e = gemm_prepare();
    if (e != cudaSuccess) return cuda_fail(e, "gemm_prepare");
    e = gemm_gws_prepare();
    if (e != cudaSuccess) return cuda_fail(e, "gemm_gws_prepare");
    e = experts_prepare();
    if (e != cudaSuccess) return cuda_fail(e, "experts_prepare");
    e = experts_umma_prepare();
    if (e != cudaSuccess) return cuda_fail(e, "experts_umma_prepare");
    e = experts_bf16_umma_prepare();
    if (e != cudaSuccess) return cuda_fail(e, "experts_bf16_umma_prepare");
    e = headtail_prepare();
    if (e != cudaSuccess) return cuda_fail(e, "headtail_prepare");
    e = segments_prepare();
    if (e != cudaSuccess) return cuda_fail(e, "segments_prepare");
    e = dense_prepare();
    if (e != cudaSuccess) return cuda_fail(e, "dense_prepare");
    e = fused_prepare();
    if (e != cudaSuccess) return cuda_fail(e, "fused_prepare");
    e = draft_prepare();
    if (e != cudaSuccess) return cuda_fail(e, "draft_prepare");
    MkModule* m = new (std::nothrow) MkModule{dev, prop.multiProcessorCount};
    MK_REQUIRE(m != nullptr, "out of host memory");
    *out = m;
    return 0;
}

void mk_module_free(MkModule* module) { delete module; }

int mk_layer_constants(const MkLayerShape* shape, MkLayerConstants* out) {
    MK_REQUIRE(out != nullptr, "out is NULL");
    if (check_shape(shape)) return -1;
    fill_constants(*shape, out);
    return 0;
}

#define NEED(field) MK_REQUIRE(b->field != 0, "bind field " #field " is 0")
#define ALIGNED16(field) MK_REQUIRE((b->field & 15) == 0, "bind field " #field " is not 16-byte aligned")

int mk_layer_bind(MkModule* module, const MkLayerShape* shape, const MkLayerBind* b, MkLaunch** out) {
    MK_REQUIRE(out != nullptr && b != nullptr, "bind or out is NULL");
    if (check_shape(shape)) return -1;
    const MkLayerShape& s = *shape;
    MkLaunch* L = new (std::nothrow) MkLaunch();
    MK_REQUIRE(L != nullptr, "out of host memory");
    struct Guard {
        MkLaunch* l;
        ~Guard() { delete l; }
    } guard{L};
    L->pack_only = module == nullptr;
    L->device = module ? module->device : -1;
    L->sms = module ? module->sms : 148;
    L->shape = s;
    L->bind = *b;
    fill_constants(s, &L->consts);
    const MkLayerConstants& c = L->consts;
    const int M = (int)s.rows, H = (int)s.hidden, P = (int)s.moe_hidden, E = (int)s.experts, K = (int)s.topk, I = (int)s.inter;
    const int qh = (int)s.q_heads, kvh = (int)s.kv_heads, G = qh / kvh, R = M * G;
    const int I_s = (int)c.inter_rank, H_s = (int)c.hidden_rank, slots = (int)c.slots;
    const int b_live = b->b_live > 0 ? (int)b->b_live : M;
    MK_REQUIRE(b_live <= M, "b_live %d exceeds rows %d", b_live, M);
    MK_REQUIRE((b->expert_lo == 0 && b->expert_hi == 0) || (b->expert_lo >= 0 && b->expert_lo < b->expert_hi && b->expert_hi <= E),
               "expert range [%lld, %lld) of %d experts", (long long)b->expert_lo, (long long)b->expert_hi, E);
    MK_REQUIRE(b->expert_hi == 0 || s.ranks == 1, "an expert range takes whole experts (ranks 1), got ranks %lld", (long long)s.ranks);
    const int ep_world = (int)b->ep_world, ep_rank = (int)b->ep_rank;
    MK_REQUIRE(ep_world == 0 || (ep_world >= 2 && ep_world <= kMaxRanks && ep_rank >= 0 && ep_rank < ep_world && b->expert_hi > 0 &&
                                 b->flags != 0 && b->w1_pack != 0 && !s.bf16),
               "an expert-parallel world needs 2..8 ranks, a rank inside it, an expert range, a flag block and the packed NVFP4 "
               "images (ep_rank %lld, ep_world %lld)", (long long)b->ep_rank, (long long)b->ep_world);
    const bool fp4 = !s.bf16, tail = s.tail != 0;

    NEED(qkv_in); NEED(k_cache); NEED(v_cache); NEED(page_table); NEED(kv_len); NEED(x_attn);
    NEED(w_o); NEED(ar); NEED(branch); NEED(stream_in); NEED(alpha); NEED(beta); NEED(prenorm_w); NEED(stream_out); NEED(h3); NEED(h3f);
    NEED(w_p); NEED(pool_ag); NEED(w_r); NEED(logits); NEED(expert_bias); NEED(topk_idx32); NEED(topk_w); NEED(gamma); NEED(q);
    NEED(z); NEED(zb); NEED(gamma_p1); NEED(y);
    MK_REQUIRE((b->w1_pack == 0) == (b->w2_pack == 0), "w1_pack and w2_pack must be bound together");
    // packed images: NVFP4 stages on an NVFP4 layer, bf16 tile images (one image per expert, weights.py pack_umma) on a
    // bf16 layer
    const bool use_umma = b->w1_pack != 0 && fp4, use_bf16_umma = b->w1_pack != 0 && !fp4;
    if (use_bf16_umma) {
        MK_REQUIRE(I_s % 64 == 0 && H_s % 128 == 0 && P % 128 == 0 && I % 128 == 0,
                   "the tensor-core bf16 experts need I/ranks a multiple of 64, P/ranks, P and I multiples of 128");
        ALIGNED16(w1_pack); ALIGNED16(w2_pack);
    } else if (use_umma) {
        MK_REQUIRE(I_s % 128 == 0 && H_s % 128 == 0 && P % 256 == 0 && I % 256 == 0 && P <= 4096 && I <= 4096,
                   "the tensor-core expert path needs I/ranks and P/ranks multiples of 128 and P, I multiples of 256 up to 4096");
        ALIGNED16(w1_pack); ALIGNED16(w2_pack);
    } else {
        NEED(w1_gate); NEED(w1_up); NEED(w2);
    }
    L->use_bf16_umma = use_bf16_umma;
    NEED(w_up); NEED(unpool_ag); NEED(c_alpha); NEED(c_beta); NEED(c_pre_w); NEED(c_post_w); NEED(c_stream_out); NEED(h3q);
    NEED(ws); NEED(status);
    if (fp4) {
        NEED(sf); NEED(x_scale); NEED(g1_alphas); NEED(g1_scale_c); NEED(g2_alphas);
        NEED(z_sf); NEED(z_ex);
        if (!use_umma) {
            NEED(w1_gate_sf); NEED(w1_up_sf); NEED(w2_sf);
        }
    }
    if (!tail) {
        NEED(w_qkv); NEED(qkv_out); NEED(cache_loc); NEED(next_k_cache); NEED(next_v_cache);
        if (s.next_rope) NEED(cos_sin);
    }
    ALIGNED16(qkv_in); ALIGNED16(k_cache); ALIGNED16(v_cache); ALIGNED16(w_o); ALIGNED16(w_p); ALIGNED16(w_r); ALIGNED16(w_up);
    ALIGNED16(w_qkv); ALIGNED16(w1_gate); ALIGNED16(w1_up); ALIGNED16(w2); ALIGNED16(h3); ALIGNED16(h3f); ALIGNED16(y);
    ALIGNED16(x_attn); ALIGNED16(h3q); ALIGNED16(q); ALIGNED16(z); ALIGNED16(ws); ALIGNED16(pool_ag); ALIGNED16(ar);
    ALIGNED16(unpool_ag); ALIGNED16(zb); ALIGNED16(w1_gate_sf); ALIGNED16(w1_up_sf); ALIGNED16(w2_sf); ALIGNED16(z_sf);
    MK_REQUIRE(c.kv_row_bytes % 16 == 0, "kv row is not a multiple of 16 bytes");
    MK_REQUIRE(b->page_stride >= M, "page_stride %lld smaller than the window", (long long)b->page_stride);
    MK_REQUIRE(b->ar_peer[s.rank] == 0 || b->ar_peer[s.rank] == b->ar, "ar_peer[rank] must be this rank's workspace");

    // peers: a present peer receives this rank's pushes; this rank's own buffer is always a destination
    auto peers = [&](const uint64_t* arr, uint64_t own, void** dst, int first, int count) {
        int n = 0;
        for (int r = first; r < first + count; ++r) {
            const uint64_t p = r == s.rank ? own : arr[r];
            if (p) dst[n++] = (void*)p;
        }
        return n;
    };
    const int node0 = (int)(s.rank - s.rank % s.node_ranks), nr = (int)s.node_ranks, jnode = (int)(s.rank % s.node_ranks);

    // exchange points: the ranks of a group that are present (own flag block and the peers' that are bound) signal and are
    // waited for; without a flag block the launches rely on stream order alone
    unsigned* const flags = (unsigned*)b->flags;
    const long long budget = b->wait_budget > 0 ? b->wait_budget : kDefaultWaitBudget;
    auto flag_of = [&](int r) -> unsigned* { return (unsigned*)(r == s.rank ? b->flags : b->flags_peer[r]); };
    // packet mode: the bf16 exchanges carry their own validity (params.h pkt_take_n); the h planes keep their counter word
    const bool packets = b->packets != 0;
    MK_REQUIRE(!packets || b->fused != 1, "packets is not available with the fused form (fused = 1)");
    auto in_band = [&](int point) { return packets && (point == XP_AR || point == XP_POOL || point == XP_ZB || point == XP_UNPOOL); };
    auto signal_to = [&](XchgSignal& x, int point, int first, int count) {
        memset(&x, 0, sizeof x);
        if (flags == nullptr || in_band(point)) return;
        for (int r = first; r < first + count; ++r)
            if (flag_of(r)) {
                x.flag[x.n++] = flag_of(r) + point;
                x.remote |= r != s.rank;
            }
        x.done = flags + kXchgDone + point;
        x.epoch = flags + kXchgEpoch + point;
    };
    auto wait_for = [&](XchgWait& w, int point, int first, int count, int stage) {
        memset(&w, 0, sizeof w);
        if (in_band(point)) {
            // the sources that are bound (own buffer and the peers' that were given) write their part; bit j: source first + j
            const uint64_t* arr = point == XP_AR ? b->ar_peer : point == XP_POOL ? b->pool_ag_peer : point == XP_ZB ? b->zb_peer : b->unpool_ag_peer;
            for (int r = first; r < first + count; ++r)
                if (r == s.rank || arr[r] != 0) w.present |= 1u << (r - first);
            w.band = point == XP_AR ? 0 : (int)((point == XP_UNPOOL ? s.hidden : s.moe_hidden) / count);
            w.packets = 1;
            w.budget = budget;
            w.status = (int*)b->status;
            w.stage = stage;
            return;
        }
        if (flags == nullptr) return;
        for (int r = first; r < first + count; ++r) w.contributors += flag_of(r) != nullptr;
        w.flag = flags + point;
        w.epoch = flags + kXchgEpoch + point;
        w.budget = budget;
        w.status = (int*)b->status;
        w.stage = stage;
    };
    const int all = (int)s.ranks, s_rank = (int)s.rank;

    // scratch carve (must follow fill_constants)
    unsigned char* ws = (unsigned char*)b->ws;
    size_t off = 0;
    float* attn_ws = (float*)(ws + off);
    off += align_up((size_t)kvh * c.attn_splits * R * 66 * 4, 256);
    float* gpart = (float*)(ws + off);
    int64_t nmax = c.qkv_row > s.hidden ? c.qkv_row : s.hidden;
    off += align_up((size_t)32 * 16 * nmax * 4, 256);
    unsigned* gcnt = (unsigned*)(ws + off);
    off += align_up((size_t)1024 * 4, 256);
    L->rt = (RouteTables*)(ws + off);
    off += align_up(sizeof(RouteTables), 256);
    L->route_ticket = gcnt + 560;  // behind the fused kernels' meeting counters
    L->z_sfd = ws + off;
    off += align_up((size_t)slots * I / 16, 256);
    L->rowscale = (float*)(ws + off);
    off += align_up((size_t)slots * 4, 256);
    unsigned char* const bf16_scratch = ws + off;
    if (s.bf16) off += align_up(kBf16UmmaScratchBytes, 256);
    MK_REQUIRE((int64_t)off == c.ws_bytes, "internal: scratch carve %zu != %lld", off, (long long)c.ws_bytes);
    L->status = (int*)b->status;
    L->max_active = slots < E ? slots : E;
    L->slots_live = b_live * K;
    for (int i = 0; i < ST_COUNT; ++i) L->stage_on[i] = true;
    L->stage_on[ST_HROW] = fp4;
    L->stage_on[ST_NQ] = L->stage_on[ST_TABLES] = false;
    L->stage_on[ST_QKV] = !tail;
    L->stage_on[ST_ROWOPS] = false;  // folded into the qkv GEMM's epilogue

    // attention
    L->attn = AttnArgs{(const bf16*)b->qkv_in, (const unsigned char*)b->k_cache, (const unsigned char*)b->v_cache,
                       (const long long*)b->page_table, (const int*)b->kv_len, attn_ws, (bf16*)b->x_attn,
                       M, qh, kvh, G, R, (int)c.qkv_row, (int)s.window, (int)c.attn_splits, (const int*)b->tree};
    // GEMMs
    (void)gpart;
    (void)gcnt;
    auto gemm = [&](GemmArgs& g, int mode, bool wf32, uint64_t w, uint64_t x, int N, int Kd, int ldw) -> int {
        memset(&g, 0, sizeof g);
        g.w = (const void*)w;
        g.x = (const void*)x;
        g.M = M; g.N = N; g.K = Kd; g.ldw = ldw; g.ldx = Kd;
        g.mode = mode;
        g.status = L->status;
        MK_REQUIRE(gemm_plan(wf32, mode, N, Kd, module ? module->sms : 148, &g.wn, &g.ksplit) == 0, "GEMM [%d x %d] has no tile / K-split plan", N, Kd);
        return 0;
    };
    // o_proj: x_attn [M, qh 64] . w_o [H, qh 64]^T -> this rank's slot of every present rank's workspace
    if (gemm(L->oproj, 0, false, b->w_o, b->x_attn, H, qh * kHeadDim, qh * kHeadDim)) return -1;
    {
        void* dst[kMaxRanks];
        const int n = peers(b->ar_peer, b->ar, dst, 0, (int)s.ranks);
        for (int i = 0; i < n; ++i) L->oproj.out[i] = (bf16*)dst[i] + (size_t)s.rank * M * H;
        L->oproj.n_out = n;
        L->oproj.ldo = H;
        L->oproj.col0 = 0;
        signal_to(L->oproj.sig, XP_AR, 0, all);
    }
    // pooler: the node block of rows [j P/nr, (j+1) P/nr) -> the node's gather rows
    // (item images hold this rank's node block only; row-major matrices are replicated and offset here)
    if (gemm(L->pooler, 0, false, b->dense_packed ? b->w_p : b->w_p + (uint64_t)jnode * (P / nr) * H * 2, b->h3, P / nr, H, H)) return -1;
    L->pooler.n_out = peers(b->pool_ag_peer, b->pool_ag, L->pooler.out, node0, nr);
    L->pooler.ldo = P;
    L->pooler.col0 = jnode * (P / nr);
    signal_to(L->pooler.sig, XP_POOL, node0, nr);
    // router: f32 weights through tf32, f32 activations, f32 logits (replicated on every rank)
    if (gemm(L->router, 0, true, b->w_r, b->h3f, E, H, H)) return -1;
    L->router.out[0] = (void*)b->logits;
    L->router.n_out = 1;
    L->router.ldo = E;
    L->router.out_f32 = 1;
    // the routing's selection scores come out of this GEMM's epilogue (a thread per logit); they live in the last
    // 16 x 1024 floats of the partial-sum scratch (the partial sums never reach that far: checked with the GEMM tiling)
    float* const scores = gpart + (size_t)512 * nmax - 16 * 1024;
    L->router.score = scores;
    L->router.score_bias = (const float*)b->expert_bias;
    L->router.score_mult = b->router_mult;
    // unpooler: node block of [H, P]
    if (gemm(L->unpool, 0, false, b->dense_packed ? b->w_up : b->w_up + (uint64_t)jnode * (H / nr) * P * 2, b->y, H / nr, P, P)) return -1;
    L->unpool.n_out = peers(b->unpool_ag_peer, b->unpool_ag, L->unpool.out, node0, nr);
    L->unpool.ldo = H;
    L->unpool.col0 = jnode * (H / nr);
    signal_to(L->unpool.sig, XP_UNPOOL, node0, nr);
    // successor's qkv
    if (!tail) {
        if (gemm(L->qkv, 1, false, b->w_qkv, b->h3q, (int)c.qkv_row, H, H)) return -1;
        L->qkv.out[0] = (void*)b->qkv_out;
        L->qkv.n_out = 1;
        L->qkv.ldo = (int)c.qkv_row;
        // the row ops ride the GEMM's epilogue (one head per tile)
        L->qkv.cos_sin = s.next_rope ? (const float*)b->cos_sin : nullptr;
        L->qkv.cache_loc = (const int*)b->cache_loc;
        L->qkv.k_cache = (unsigned char*)b->next_k_cache;
        L->qkv.v_cache = (unsigned char*)b->next_v_cache;
        L->qkv.q_scale = (float)b->q_scale;
        L->qkv.eps = (float)b->qkv_eps;
        L->qkv.qh = qh;
        L->qkv.kvh = kvh;
        L->qkv.kv_row_bytes = (int)c.kv_row_bytes;
    }
    // norms
    L->post_norm = NormArgs{0, H, (int)s.ranks, (const bf16*)b->ar, (bf16*)b->branch, (const float*)b->stream_in,
                            (const float*)b->alpha, (const float*)b->beta, (const bf16*)b->prenorm_w, nullptr,
                            (float*)b->stream_out, (bf16*)b->h3, (float*)b->h3f, M};
    L->cross_norm = NormArgs{1, H, (int)s.ranks, (const bf16*)b->unpool_ag, nullptr, (const float*)b->stream_out,
                             (const float*)b->c_alpha, (const float*)b->c_beta, (const bf16*)b->c_pre_w, (const bf16*)b->c_post_w,
                             (float*)b->c_stream_out, (bf16*)b->h3q, nullptr, M};
    wait_for(L->post_norm.wait, XP_AR, 0, all, ST_POST_NORM);
    wait_for(L->cross_norm.wait, XP_UNPOOL, node0, nr, ST_CROSS_NORM);
    L->topk = TopkArgs{(const float*)b->logits, (const float*)b->expert_bias, (int*)b->topk_idx32, (float*)b->topk_w,
                       b->router_mult, (float)b->route_scale, E, K, M, (int*)b->status, scores, (int)b->expert_lo, (int)b->expert_hi};
    L->nq = NqArgs{(const bf16*)b->pool_ag, (const bf16*)b->gamma, (unsigned char*)b->q, (unsigned char*)b->sf,
                   (float*)b->x_scale, (float)b->eps, P, (int)s.bf16};
    L->combine = CombineArgs{(const bf16*)b->zb, (const float*)b->topk_w, (const bf16*)b->gamma_p1, (bf16*)b->y, P, K, b_live};
    wait_for(L->nq.wait, XP_POOL, node0, nr, ST_NQ);
    wait_for(L->combine.wait, XP_ZB, 0, all, ST_COMBINE);
    wait_for(L->hrow_wait, XP_Z, 0, all, ST_HROW);
    L->rowops = RowopsArgs{(bf16*)b->qkv_out, s.next_rope ? (const float*)b->cos_sin : nullptr, (const int*)b->cache_loc,
                           (unsigned char*)b->next_k_cache, (unsigned char*)b->next_v_cache, (float)b->q_scale, (float)b->qkv_eps,
                           M, qh, kvh, (int)c.qkv_row, (int)c.kv_row_bytes};
    // experts
    ExpertArgs& ex = L->ex;
    memset(&ex, 0, sizeof ex);
    ex.rt = L->rt;
    ex.P = P; ex.I = I; ex.I_s = I_s; ex.H_s = H_s; ex.rank = (int)s.rank; ex.ranks = (int)s.ranks; ex.topk = K; ex.wbf16 = (int)s.bf16;
    ex.xq = (const unsigned char*)b->q;
    ex.x_sf = (const unsigned char*)b->sf;
    ex.x_scale = (const float*)b->x_scale;
    ex.w1_gate = (const unsigned char*)b->w1_gate;
    ex.w1_gate_sf = (const unsigned char*)b->w1_gate_sf;
    ex.w1_up = (const unsigned char*)b->w1_up;
    ex.w1_up_sf = (const unsigned char*)b->w1_up_sf;
    ex.g1_alphas = (const float*)b->g1_alphas;
    ex.g1_scale_c = (const float*)b->g1_scale_c;
    ex.n_peer = peers(b->z_peer, b->z, (void**)ex.z_peer, 0, (int)s.ranks);
    if (fp4) {
        const int n1 = peers(b->zsf_peer, b->z_sf, (void**)ex.zsf_peer, 0, (int)s.ranks);
        const int n2 = peers(b->zex_peer, b->z_ex, (void**)ex.zex_peer, 0, (int)s.ranks);
        MK_REQUIRE(n1 == ex.n_peer && n2 == ex.n_peer, "z_peer / zsf_peer / zex_peer name different ranks");
    }
    {
        const int n3 = peers(b->zb_peer, b->zb, (void**)ex.zb_peer, 0, (int)s.ranks);
        MK_REQUIRE(n3 == ex.n_peer, "zb_peer and z_peer name different ranks");
    }
    ex.z = (const unsigned char*)b->z;
    ex.z_sfd = L->z_sfd;
    ex.rowscale = L->rowscale;
    ex.w2 = (const unsigned char*)b->w2;
    ex.w2_sf = (const unsigned char*)b->w2_sf;
    ex.g2_alphas = (const float*)b->g2_alphas;
    signal_to(ex.sig_g1, XP_Z, 0, all);
    signal_to(ex.sig_g2, XP_ZB, 0, all);
    if (!fp4) wait_for(ex.wait_g2, XP_Z, 0, all, ST_G2);  // no h-row kernel in a bf16 layer: g2 itself waits
    MK_REQUIRE(g1_smem(P) <= 200 * 1024 && g2_smem(I) <= 200 * 1024, "expert rows exceed shared memory");
    L->use_umma = use_umma;
    L->sms = module ? module->sms : 148;
    if (use_bf16_umma) {
        MK_REQUIRE(L->sms <= kBf16UmmaMaxGrid, "%d CTAs exceed the grouped experts' scratch", L->sms);
        for (int g2 = 0; g2 < 2; ++g2) {
            Bf16UmmaArgs& u = g2 ? L->bf16_g2 : L->bf16_g1;
            memset(&u, 0, sizeof u);
            u.rt = L->rt;
            u.w = (const unsigned char*)(g2 ? b->w2_pack : b->w1_pack);
            u.x = (const bf16*)(g2 ? b->z : b->q);
            u.K = g2 ? I : P;
            u.NB = g2 ? H_s / 128 : 2 * I_s / 128;
            u.topk = K;
            u.by_token = !g2;
            u.g2 = g2;
            for (int i = 0; i < ex.n_peer; ++i) u.out[i] = g2 ? ex.zb_peer[i] : (bf16*)ex.z_peer[i];
            u.n_out = ex.n_peer;
            u.ldo = g2 ? P : I;
            u.col0 = (long long)s.rank * (g2 ? H_s : I_s);
            u.part = (float*)bf16_scratch;
            u.ticket = (unsigned*)(bf16_scratch + (size_t)2 * kBf16UmmaMaxGrid * 2048 * 4) + (g2 ? kBf16UmmaMaxGrid : 0);
            if (g2) u.wait = ex.wait_g2;
            u.sig = g2 ? ex.sig_g2 : ex.sig_g1;
            u.status = L->status;
        }
    }
    if (use_umma) {
        for (int g2 = 0; g2 < 2; ++g2) {
            UmmaArgs& u = g2 ? L->umma_g2 : L->umma_g1;
            memset(&u, 0, sizeof u);
            u.rt = L->rt;
            u.K = g2 ? I : P;
            u.NB = (g2 ? H_s : I_s) / 128;
            u.P = P; u.I = I; u.I_s = I_s; u.H_s = H_s; u.rank = (int)s.rank; u.topk = K;
            u.wpack = (const unsigned char*)(g2 ? b->w2_pack : b->w1_pack);
            u.bq = g2 ? (const unsigned char*)b->z : (const unsigned char*)b->q;
            // g2 forms the h-row view in its own stager (row exponents, moved scale bytes, row scales): no h-row kernel
            u.bsf = g2 ? (const unsigned char*)b->z_sf : (const unsigned char*)b->sf;
            u.bex = g2 ? (const signed char*)b->z_ex : nullptr;
            if (g2) {
                u.wait = L->hrow_wait;
                // packet mode: g2 orders itself behind g1 by the h planes' counter word alone (g1 announces the epoch)
                u.wait.packets = packets && u.wait.flag != nullptr;
                if (u.wait.packets) u.wait.target = flags + kXchgTarget + XP_Z;
            }
            u.x_scale = (const float*)b->x_scale;
            u.g1_alphas = (const float*)b->g1_alphas;
            u.g1_scale_c = (const float*)b->g1_scale_c;
            u.rowscale = L->rowscale;
            u.g2_alphas = (const float*)b->g2_alphas;
            for (int i = 0; i < ex.n_peer; ++i) {
                u.z_peer[i] = ex.z_peer[i];
                u.zsf_peer[i] = ex.zsf_peer[i];
                u.zex_peer[i] = ex.zex_peer[i];
                u.zb_peer[i] = ex.zb_peer[i];
            }
            u.n_peer = ex.n_peer;
            u.status = L->status;
            u.sig = g2 ? ex.sig_g2 : ex.sig_g1;
            if (!g2 && packets && u.sig.n > 0) u.sig.target = flags + kXchgTarget + XP_Z;
        }
        if (ep_world > 1) {
            // whole experts per rank, one process per GPU: the h planes stay local, the zb rows of this rank's (row, slot)
            // pairs go to every rank of the expert-parallel world, whose combines wait for all of them
            UmmaArgs& u = L->umma_g2;
            u.n_peer = 0;
            memset(&u.sig, 0, sizeof u.sig);
            for (int r = 0; r < ep_world; ++r) {
                const uint64_t zb = r == ep_rank ? b->zb : b->zb_peer[r], fl = r == ep_rank ? b->flags : b->flags_peer[r];
                MK_REQUIRE(zb != 0 && (packets || fl != 0), "zb_peer[%d] or flags_peer[%d] of the expert-parallel world is 0", r, r);
                u.zb_peer[u.n_peer++] = (bf16*)zb;
                u.sig.flag[u.sig.n++] = (unsigned*)fl + XP_ZB;
                u.sig.remote |= r != ep_rank;
            }
            u.sig.done = flags + kXchgDone + XP_ZB;
            u.sig.epoch = flags + kXchgEpoch + XP_ZB;
            XchgWait& w = L->combine.wait;
            memset(&w, 0, sizeof w);
            w.budget = budget;
            w.status = (int*)b->status;
            w.stage = ST_COMBINE;
            if (packets) {  // whole rows from whichever rank owns the slot's expert: every packet of a live row arrives
                memset(&u.sig, 0, sizeof u.sig);
                w.packets = 1;
                w.present = (1u << ep_world) - 1;
                w.band = 0;
            } else {
                w.flag = flags + XP_ZB;
                w.epoch = flags + kXchgEpoch + XP_ZB;
                w.contributors = (unsigned)ep_world;
            }
        }
        L->stage_on[ST_HROW] = false;
    }
    // The fused form of the dense stages (segments.cuh): two persistent kernels with grid barriers. Its exchange waits
    // poll for peers that run at the same time, so it serves a lone rank or one process per GPU; a world emulated on one
    // GPU steps the per-stage kernels (mk_launch_step) instead. Shapes outside its tiling keep the per-stage kernels.
    L->use_segments = false;
    L->seg_gemms = false;
    const size_t part_cap = (size_t)512 * nmax - 16 * 1024;  // floats of partial-sum scratch below the routing scores
    const bool seg_shapes = (qh * kHeadDim) % 512 == 0 && H % 512 == 0 && P % 512 == 0 && H <= 8192 && P <= 4096 &&
                            (size_t)(H / 256) * 16 * (P / nr + E) <= part_cap &&
                            (size_t)(qh * kHeadDim / 256) * 16 * H <= part_cap && (size_t)(P / 256) * 16 * (H / nr) <= part_cap &&
                            (size_t)(H / 256) * 16 * c.qkv_row <= part_cap;
    auto seg_gemm = [&](SegGemm& g, const GemmArgs& src, bool f32, float* part) {
        const int es = f32 ? 4 : 2;
        g.w = (const unsigned char*)src.w;
        g.x = (const unsigned char*)src.x;
        g.ldw = (long long)src.ldw * es;
        g.ldx = (long long)src.ldx * es;
        g.N = src.N; g.K = src.K; g.M = src.M; g.f32 = f32 ? 1 : 0;
        g.part = part;
        g.packed = (int)b->dense_packed;
    };
    // fused 0 (default): the per-stage launch list with its GEMMs on the item engine of segments.cuh where the shapes tile
    // (pooler and router share a launch); fused 2: the cluster split-K GEMMs of gemm.cu everywhere; fused 1: two segments
    // dense_packed 2: tile images of the tcgen05 engine (dense.cu): every K a whole number of 256-byte stages
    const bool umma_images = b->dense_packed == 2;
    const bool umma_shapes = (qh * kHeadDim) % 128 == 0 && H % 128 == 0 && P % 128 == 0;
    MK_REQUIRE(b->dense_packed >= 0 && b->dense_packed <= 2, "dense_packed %lld is not 0, 1 or 2", (long long)b->dense_packed);
    MK_REQUIRE(b->dense_packed != 1 || (b->fused != 2 && seg_shapes), "dense_packed 1 needs the item engine (fused 0 or 1 and shapes it tiles)");
    MK_REQUIRE(!umma_images || (b->fused != 2 && umma_shapes),
               "dense_packed 2 needs fused 0 or 1 and K dimensions that are multiples of 128");
    MK_REQUIRE(!(umma_images && b->fused == 1) || (H % 1024 == 0 && P <= 4096 && K <= 8),
               "the fused tensor-core kernels need hidden a multiple of 1024, moe_hidden <= 4096 and topk <= 8");
    if (umma_images || (b->fused != 2 && seg_shapes)) {
        L->seg_gemms = true;
        const GridBarrier gb{(unsigned long long*)gcnt, budget, L->status};
        auto stage = [&](SegGemmArgs& g, const GemmArgs& src, int finish) {
            memset(&g, 0, sizeof g);
            seg_gemm(g.g[0], src, false, gpart);
            g.n_gemm = 1;
            g.finish = finish;
            for (int i = 0; i < src.n_out; ++i) g.out[i] = (bf16*)src.out[i];
            g.n_out = src.n_out;
            g.ldo = src.ldo;
            g.off0 = src.col0;
            g.sig = src.sig;
            g.gb = gb;
            g.status = L->status;
        };
        stage(L->sg_oproj, L->oproj, 0);
        stage(L->sg_pool, L->pooler, 1);
        seg_gemm(L->sg_pool.g[1], L->router, true, gpart + (size_t)(H / 256) * 16 * (P / nr));
        L->sg_pool.n_gemm = 2;
        L->sg_pool.f32_out = (float*)b->logits;
        // tile images: the routing kernel forms the selection scores itself (a thread per logit) instead of the CTA that
        // finishes a router tile (a row's worth of f64 sigmoids per thread at the tail of the GEMM)
        L->sg_pool.score = umma_images ? nullptr : scores;
        if (umma_images) L->topk.score = nullptr;
        L->sg_pool.score_bias = (const float*)b->expert_bias;
        L->sg_pool.score_mult = b->router_mult;
        stage(L->sg_unpool, L->unpool, 0);
        if (!tail) {
            stage(L->sg_qkv, L->qkv, 2);
            L->sg_qkv.epi = L->qkv;
        }
        L->stage_on[ST_ROUTER] = false;  // rides the pooler's launch
        if (umma_images) {
            // stream-K partial sums below the routing scores, tickets behind the grid-barrier word
            unsigned* const tickets = gcnt + 64;
            SegGemmArgs* all4[4] = {&L->sg_oproj, &L->sg_pool, &L->sg_unpool, tail ? nullptr : &L->sg_qkv};
            for (SegGemmArgs* g : all4)
                MK_REQUIRE(g == nullptr || dense_setup(*g, L->sms, gpart, part_cap, tickets, 448 - 64),
                           "a dense GEMM of this shape does not fit the tensor-core engine's scratch");
        }
    }
    L->use_fused = false;
    if (b->fused == 1 && umma_images) {
        // The fused form on the tensor-core engine (fused.cuh): kernel A = o_proj .. routing, kernel B = combine .. qkv head.
        // Like the segment kernels its exchange waits poll for peers that run at the same time: a lone rank or one process
        // per GPU; mk_launch_step still runs the per-stage kernels.
        L->use_fused = true;
        // the 1024 counter words: [0, 2) grid barrier, [16, 48) the two kernels' launch / dependency words, [64, 448) tile
        // tickets, [448, 544) the row meetings' counters of kernels A and B; the meetings' partial sums take the last 2048
        // floats of the partial-sum scratch
        unsigned* const words = gcnt + 16;
        unsigned* const tickets = gcnt + 64;
        const size_t ticket_cap = 448 - 64;
        const int norm_parts = H / 1024, combine_parts = (P + 1023) / 1024;
        MK_REQUIRE(norm_parts <= 8 && combine_parts <= 4, "the fused kernels cut a row into at most 8 (hidden) / 4 (moe_hidden) parts");
        auto units = [](const SegGemm& g) { return (long long)((g.N + 127) / 128) * (g.K * (g.f32 ? 4 : 2) / 256); };
        auto grid_for = [&](const SegGemmArgs& x, const SegGemmArgs* y) {
            long long G = L->sms < 148 ? L->sms : 148;
            const long long t0 = units(x.g[0]) + (x.n_gemm > 1 ? units(x.g[1]) : 0);
            if (t0 < G) G = t0;
            if (y != nullptr) {
                const long long t1 = units(y->g[0]) + (y->n_gemm > 1 ? units(y->g[1]) : 0);
                if (t1 < G) G = t1;
            }
            return (int)G;
        };
        auto fused_wait = [&](FusedArgs& F, int s, int point, int first, int count, int tiles, int stage) {
            F.wait_flag[s] = nullptr;
            F.wait_epoch[s] = nullptr;
            F.bump_epoch[s] = nullptr;
            F.wait_contrib[s] = 0;
            F.wait_stage[s] = stage;
            XchgSignal& x = s == 0 ? F.sig0 : F.sig1;
            memset(&x, 0, sizeof x);
            if (flags == nullptr || point < 0) return;
            unsigned present = 0;
            for (int r = first; r < first + count; ++r)
                if (flag_of(r)) {
                    x.flag[x.n++] = flag_of(r) + kFusedFlag + point;
                    x.remote |= r != s_rank;
                    ++present;
                }
            F.wait_flag[s] = flags + kFusedFlag + point;
            F.wait_epoch[s] = flags + kFusedEpoch + point;
            F.bump_epoch[s] = flags + kFusedEpoch + point;
            F.wait_contrib[s] = present * (unsigned)tiles;
        };
        FusedArgs& A = L->fused_a;
        memset(&A, 0, sizeof A);
        A.st[0] = L->sg_oproj;
        A.st[1] = L->sg_pool;
        A.st[0].sig = XchgSignal{};
        A.st[1].sig = XchgSignal{};
        A.st[1].score = nullptr;  // the top-k CTAs compute the selection scores (spread over their threads)
        A.score_out = scores;
        A.n_stages = 2;
        A.row_kind[0] = 0; A.row_kind[1] = 1; A.row_kind[2] = 2;
        A.M = M;
        A.norm = L->post_norm;
        A.topk = L->topk;
        A.nq = L->nq;
        A.rt = L->rt;
        A.b_live = b_live;
        A.launches = words; A.done = words + 1; A.dep = words + 2;
        A.norm_parts = norm_parts; A.combine_parts = combine_parts;
        const size_t fused_cap = part_cap - 2048;
        A.meet_count = gcnt + 448; A.meet_part = gpart + fused_cap;
        A.tiles0[0] = (H + 127) / 128;
        A.tiles0[1] = (P / nr + 127) / 128;
        A.router_tiles = (E + 127) / 128;
        fused_wait(A, 0, XP_AR, 0, all, A.tiles0[0], ST_POST_NORM);
        fused_wait(A, 1, XP_POOL, node0, nr, A.tiles0[1], ST_NQ);
        A.budget = budget;
        A.status = L->status;
        L->fused_grid_a = grid_for(A.st[0], &A.st[1]);
        MK_REQUIRE(L->fused_grid_a >= M * norm_parts && L->fused_grid_a > M,
                   "the fused kernel A has %d CTAs for %d row parts and the routing", L->fused_grid_a, M * norm_parts);
        MK_REQUIRE(dense_setup(A.st[0], L->sms, gpart, fused_cap, tickets, ticket_cap, L->fused_grid_a) &&
                       dense_setup(A.st[1], L->sms, gpart, fused_cap, tickets, ticket_cap, L->fused_grid_a),
                   "a dense GEMM of this shape does not fit the fused kernel's scratch");
        {
            // the CTAs that hold a K range of a router tile (the kernel's own cut: unit s belongs to the largest c with
            // floor(c T / G) <= s)
            const long long T0 = units(A.st[1].g[0]), T = T0 + units(A.st[1].g[1]), G = L->fused_grid_a;
            const long long KS = (long long)H * 4 / 256;
            auto cta_of = [&](long long u) { return ((u + 1) * G + T - 1) / T - 1; };
            long long total = 0;
            for (int t = 0; t < A.router_tiles; ++t) total += cta_of(T0 + (t + 1) * KS - 1) - cta_of(T0 + t * KS) + 1;
            A.router_contribs = (int)total;
        }
        FusedArgs& B = L->fused_b;
        memset(&B, 0, sizeof B);
        B.st[0] = L->sg_unpool;
        B.st[0].sig = XchgSignal{};
        B.n_stages = 1;
        if (!tail) {
            B.st[1] = L->sg_qkv;
            B.st[1].sig = XchgSignal{};
            B.n_stages = 2;
        }
        B.row_kind[0] = 3; B.row_kind[1] = 1; B.row_kind[2] = 0;
        B.M = M;
        B.norm = L->cross_norm;
        B.combine = L->combine;
        B.b_live = b_live;
        B.launches = words + 8; B.done = words + 9; B.dep = words + 10;
        B.norm_parts = norm_parts; B.combine_parts = combine_parts;
        B.meet_count = gcnt + 496; B.meet_part = gpart + fused_cap + 1024;
        B.tiles0[0] = (H / nr + 127) / 128;
        B.tiles0[1] = tail ? 0 : ((int)c.qkv_row + 127) / 128;
        fused_wait(B, 0, XP_UNPOOL, node0, nr, B.tiles0[0], ST_CROSS_NORM);
        fused_wait(B, 1, -1, 0, 0, 0, 0);
        B.budget = budget;
        B.status = L->status;
        L->fused_grid_b = grid_for(B.st[0], tail ? nullptr : &B.st[1]);
        MK_REQUIRE(L->fused_grid_b >= M * norm_parts && L->fused_grid_b >= M * combine_parts,
                   "the fused kernel B has %d CTAs for %d / %d row parts", L->fused_grid_b, M * norm_parts, M * combine_parts);
        MK_REQUIRE(dense_setup(B.st[0], L->sms, gpart, fused_cap, tickets, ticket_cap, L->fused_grid_b) &&
                       (tail || dense_setup(B.st[1], L->sms, gpart, fused_cap, tickets, ticket_cap, L->fused_grid_b)),
                   "a dense GEMM of this shape does not fit the fused kernel's scratch");
    }
    if (b->fused == 1 && seg_shapes && !umma_images) {
        L->use_segments = true;
        const GridBarrier gb{(unsigned long long*)gcnt, budget, L->status};
        SegAArgs& A = L->seg_a;
        memset(&A, 0, sizeof A);
        seg_gemm(A.oproj, L->oproj, false, gpart);
        seg_gemm(A.pooler, L->pooler, false, gpart);
        seg_gemm(A.router, L->router, true, gpart + (size_t)(H / 256) * 16 * (P / nr));
        for (int i = 0; i < L->oproj.n_out; ++i) A.ar_out[i] = (bf16*)L->oproj.out[i];
        A.n_ar = L->oproj.n_out;
        A.ar_off = 0;  // the destinations already point at this rank's slot
        A.sig_ar = L->oproj.sig;
        A.post_norm = L->post_norm;
        for (int i = 0; i < L->pooler.n_out; ++i) A.pool_out[i] = (bf16*)L->pooler.out[i];
        A.n_pool = L->pooler.n_out;
        A.pool_ld = L->pooler.ldo;
        A.pool_col0 = L->pooler.col0;
        A.sig_pool = L->pooler.sig;
        A.logits = (float*)b->logits;
        A.topk = L->topk;
        A.topk.score = nullptr;  // the segment's routing stage computes the scores itself
        A.nq = L->nq;
        A.rt = L->rt;
        A.b_live = b_live;
        A.gb = gb;
        A.status = L->status;
        SegBArgs& B = L->seg_b;
        memset(&B, 0, sizeof B);
        B.combine = L->combine;
        B.M = M;
        seg_gemm(B.unpool, L->unpool, false, gpart);
        for (int i = 0; i < L->unpool.n_out; ++i) B.unpool_out[i] = (bf16*)L->unpool.out[i];
        B.n_unpool = L->unpool.n_out;
        B.unpool_ld = L->unpool.ldo;
        B.unpool_col0 = L->unpool.col0;
        B.sig_unpool = L->unpool.sig;
        B.cross_norm = L->cross_norm;
        B.tail = tail ? 1 : 0;
        if (!tail) {
            seg_gemm(B.qkv, L->qkv, false, gpart);
            B.qkv_epi = L->qkv;
        }
        B.gb = gb;
        B.status = L->status;
    }
    *out = L;
    guard.l = nullptr;
    return 0;
}

static int run_stage(const MkLaunch* L, int st, cudaStream_t s, bool pdl) {
    if (!L->stage_on[st]) return 0;
    cudaError_t e = cudaSuccess;
    switch (st) {
        case ST_ATTN_SPLIT: e = attn_split_launch(L->attn, s, pdl); break;
        case ST_ATTN_COMBINE: e = attn_combine_launch(L->attn, s, pdl); break;
        case ST_OPROJ: e = L->seg_gemms ? seg_gemm_launch(L->sg_oproj, L->sms, s, pdl) : gemm_launch(L->oproj, false, s, pdl); break;
        case ST_POST_NORM: e = resid_norm_launch(L->post_norm, s, pdl); break;
        case ST_POOLER: e = L->seg_gemms ? seg_gemm_launch(L->sg_pool, L->sms, s, pdl) : gemm_launch(L->pooler, false, s, pdl); break;
        case ST_ROUTER: e = gemm_launch(L->router, true, s, pdl); break;
        case ST_TOPK:  // top-k, route tables and the pre-expert norm + quantisation share one launch
            e = route_nq_launch(L->topk, L->nq, L->rt, L->combine.b_live, L->route_ticket, s, pdl);
            break;
        case ST_NQ:
        case ST_TABLES:
            break;  // folded into ST_TOPK's launch (the slots stay in the stage list: stage indices are ABI)
        case ST_G1:
            e = L->use_umma        ? experts_umma_launch(L->umma_g1, false, L->sms, s, pdl)
                : L->use_bf16_umma ? experts_bf16_umma_launch(L->bf16_g1, L->sms, s, pdl)
                                   : g1_launch(L->ex, L->max_active, s, pdl);
            break;
        case ST_HROW:
            e = hrow_launch((const unsigned char*)L->bind.z_sf, (const signed char*)L->bind.z_ex, (int)L->shape.inter / 16,
                            L->slots_live, (int)L->consts.slots, L->z_sfd, L->rowscale, L->hrow_wait, s, pdl);
            break;
        case ST_G2:
            e = L->use_umma        ? experts_umma_launch(L->umma_g2, true, L->sms, s, pdl)
                : L->use_bf16_umma ? experts_bf16_umma_launch(L->bf16_g2, L->sms, s, pdl)
                                   : g2_launch(L->ex, L->max_active, s, pdl);
            break;
        case ST_COMBINE: e = combine_launch(L->combine, (int)L->shape.rows, s, pdl); break;
        case ST_UNPOOL: e = L->seg_gemms ? seg_gemm_launch(L->sg_unpool, L->sms, s, pdl) : gemm_launch(L->unpool, false, s, pdl); break;
        case ST_CROSS_NORM: e = resid_norm_launch(L->cross_norm, s, pdl); break;
        case ST_QKV:
            e = L->is_head     ? gemm_gws_launch(L->head_gemm, false, L->head_ks, s, pdl)
                : L->seg_gemms ? seg_gemm_launch(L->sg_qkv, L->sms, s, pdl)
                               : gemm_launch(L->qkv, false, s, pdl);
            break;
        case ST_ROWOPS: e = rowops_launch(L->rowops, s, pdl); break;
        default: return fail("stage %d does not exist", st);
    }
    if (e != cudaSuccess) return fail("stage %d launch: %s", st, cudaGetErrorString(e));
    return 0;
}

static int run_dops(const MkLaunch* L, int first, int last, cudaStream_t s, bool pdl) {
    for (int i = first; i < last; ++i) {
        const DraftOp& op = L->dops[i];
        cudaError_t e = cudaSuccess;
        switch (op.kind) {
            case DOP_FEATS: e = dfeats_launch(op.feats, s, pdl); break;
            case DOP_GEMM: e = seg_gemm_launch(op.gemm, L->sms, s, pdl); break;
            case DOP_NORM: e = dnorm_launch(op.norm, s, pdl); break;
            case DOP_CONV: e = dconv_launch(op.conv, s, pdl); break;
            case DOP_QKV_ROWS: e = dqkv_rows_launch(op.rows, s, pdl); break;
            case DOP_CTX_KV: e = dctx_kv_launch(op.ckv, s, pdl); break;
            case DOP_ATTN_SPLIT: e = dattn_split_launch(op.attn, s, pdl); break;
            case DOP_ATTN_MERGE: e = dattn_merge_launch(op.attn, s, pdl); break;
            case DOP_TOPK: e = dtopk_launch(op.topk, s, pdl); break;
            case DOP_LATTICE: e = dlattice_launch(op.lat, s, pdl); break;
            case DOP_KV_SYNC: e = dkv_sync_launch(op.sync, s, pdl); break;
            case DOP_TREE: e = dtree_walk_launch(op.tree, s, pdl); break;
            case DOP_COMPACT: e = tree_compact_launch(op.compact, s, pdl); break;
            default: return fail("draft kernel kind %d does not exist", op.kind);
        }
        if (e != cudaSuccess) return fail("draft kernel %d (kind %d) launch: %s", i, op.kind, cudaGetErrorString(e));
    }
    return 0;
}

int mk_launch_step(const MkLaunch* launch, uint64_t stream, int64_t first, int64_t count) {
    MK_REQUIRE(launch != nullptr, "launch is NULL");
    MK_REQUIRE(!launch->pack_only, "a pack-only record (bound without a module) cannot launch");
    if (launch->n_dops > 0) {  // a draft launch: its kernels by index
        MK_REQUIRE(first >= 0 && count >= 0 && first + count <= launch->n_dops, "kernels [%lld, %lld) outside 0..%d", (long long)first,
                   (long long)(first + count), launch->n_dops);
        return run_dops(launch, (int)first, (int)(first + count), (cudaStream_t)stream, false);
    }
    MK_REQUIRE(launch->n_ops == 0, "mk_launch_step addresses the stages of a layer launch");
    MK_REQUIRE(first >= 0 && count >= 0 && first + count <= ST_COUNT, "stages [%lld, %lld) outside 0..%d", (long long)first,
               (long long)(first + count), ST_COUNT);
    for (int st = (int)first; st < first + count; ++st)
        if (run_stage(launch, st, (cudaStream_t)stream, false)) return -1;
    return 0;
}

static int run_ops(const MkLaunch* L, cudaStream_t s, bool pdl) {
    for (int i = 0; i < L->n_ops; ++i) {
        cudaError_t e = cudaSuccess;
        switch (L->op_kind[i]) {
            case OP_FEEDS: e = feeds_launch(L->feeds, s, pdl); break;
            case OP_ENTRY: e = entry_launch(L->entry, s, pdl); break;
            case OP_GEMM_BF16: e = gemm_launch(L->op_gemm, false, s, pdl); break;
            case OP_SOFTCAP: e = softcap_launch(L->softcap, s, pdl); break;
            case OP_ACCEPT: e = accept_launch(L->accept, s, pdl); break;
            default: return fail("op %d does not exist", L->op_kind[i]);
        }
        if (e != cudaSuccess) return fail("op %d launch: %s", L->op_kind[i], cudaGetErrorString(e));
    }
    return 0;
}

int mk_launch(const MkLaunch* launch, uint64_t stream, int pdl) {
    MK_REQUIRE(launch != nullptr, "launch is NULL");
    MK_REQUIRE(!launch->pack_only, "a pack-only record (bound without a module) cannot launch");
    if (launch->n_dops > 0) return run_dops(launch, 0, launch->n_dops, (cudaStream_t)stream, pdl != 0);
    if (launch->n_ops > 0) return run_ops(launch, (cudaStream_t)stream, pdl != 0);
    if (launch->use_fused) {
        const MkLaunch* L = launch;
        cudaStream_t s = (cudaStream_t)stream;
        const bool p = pdl != 0;
        if (run_stage(L, ST_ATTN_SPLIT, s, p) || run_stage(L, ST_ATTN_COMBINE, s, p)) return -1;
        cudaError_t e = fused_launch(L->fused_a, L->fused_grid_a, s, p);
        if (e != cudaSuccess) return fail("fused kernel A launch: %s", cudaGetErrorString(e));
        if (run_stage(L, ST_G1, s, p) || run_stage(L, ST_HROW, s, p) || run_stage(L, ST_G2, s, p)) return -1;
        e = fused_launch(L->fused_b, L->fused_grid_b, s, p);
        if (e != cudaSuccess) return fail("fused kernel B launch: %s", cudaGetErrorString(e));
        return 0;
    }
    if (launch->use_segments) {
        const MkLaunch* L = launch;
        cudaStream_t s = (cudaStream_t)stream;
        const bool p = pdl != 0;
        if (run_stage(L, ST_ATTN_SPLIT, s, p) || run_stage(L, ST_ATTN_COMBINE, s, p)) return -1;
        cudaError_t e = seg_a_launch(L->seg_a, L->sms, s, p);
        if (e != cudaSuccess) return fail("segment A launch: %s", cudaGetErrorString(e));
        if (run_stage(L, ST_G1, s, p) || run_stage(L, ST_HROW, s, p) || run_stage(L, ST_G2, s, p)) return -1;
        e = seg_b_launch(L->seg_b, L->sms, s, p);
        if (e != cudaSuccess) return fail("segment B launch: %s", cudaGetErrorString(e));
        return 0;
    }
    for (int st = 0; st < ST_COUNT; ++st)
        if (run_stage(launch, st, (cudaStream_t)stream, pdl != 0)) return -1;
    return 0;
}

void mk_launch_free(MkLaunch* launch) {
    if (launch != nullptr) delete[] launch->dops;
    delete launch;
}

int mk_launch_params(const MkLaunch* launch, char* text, uint64_t cap_bytes) {
    MK_REQUIRE(launch != nullptr && text != nullptr, "launch or text is NULL");
    const MkLaunch* L = launch;
    MK_REQUIRE(L->n_dops == 0 && L->n_ops == 0, "not a layer launch");
    size_t n = 0;
    bool full = false;
    auto put = [&](const char* fmt, ...) {
        if (full) return;
        va_list ap;
        va_start(ap, fmt);
        const int k = vsnprintf(text + n, cap_bytes - n, fmt, ap);
        va_end(ap);
        if (k < 0 || (size_t)k >= cap_bytes - n) full = true;
        else n += (size_t)k;
    };
    auto wait = [&](const char* name, const XchgWait& w) {
        put("%s wait=%s present=0x%x band=%d contributors=%u target=%d\n", name,
            w.packets && w.flag == nullptr ? "packets" : w.flag != nullptr ? "counter" : "off", w.present, w.band, w.contributors,
            w.target != nullptr ? 1 : 0);
    };
    auto sig = [&](const char* name, const XchgSignal& x) {
        put("%s signal=%d remote=%d target=%d\n", name, x.n, x.remote, x.target != nullptr ? 1 : 0);
    };
    unsigned on = 0;
    for (int i = 0; i < ST_COUNT; ++i) on |= (L->stage_on[i] ? 1u : 0u) << i;
    put("stages on=0x%x fused=%d segments=%d\n", on, L->use_fused ? 1 : 0, L->use_segments ? 1 : 0);
    sig("o_proj", L->seg_gemms ? L->sg_oproj.sig : L->oproj.sig);
    wait("post_norm", L->post_norm.wait);
    sig("pooler", L->seg_gemms ? L->sg_pool.sig : L->pooler.sig);
    wait("nq", L->nq.wait);
    sig("g1", L->use_umma ? L->umma_g1.sig : L->ex.sig_g1);
    wait("g2", L->use_umma ? L->umma_g2.wait : L->hrow_wait);
    sig("g2", L->use_umma ? L->umma_g2.sig : L->ex.sig_g2);
    wait("combine", L->combine.wait);
    sig("unpooler", L->seg_gemms ? L->sg_unpool.sig : L->unpool.sig);
    wait("cross_norm", L->cross_norm.wait);
    MK_REQUIRE(!full, "text of %llu bytes is too small", (unsigned long long)cap_bytes);
    return (int)n;
}

int mk_launch_info(const MkLaunch* launch, MkLaunchInfo* out) {
    MK_REQUIRE(launch != nullptr && out != nullptr, "launch or out is NULL");
    const MkLaunch* L = launch;
    if (L->n_dops > 0) {
        memset(out, 0, sizeof *out);
        out->kernels = L->n_dops;
        out->grid = L->sms;
        out->block = 512;
        out->cluster = 1;
        out->smem = (int64_t)segments_smem();
        out->param_bytes = (int64_t)sizeof(MkLaunch) + (int64_t)L->n_dops * (int64_t)sizeof(DraftOp);
        return 0;
    }
    if (L->n_ops > 0) {
        memset(out, 0, sizeof *out);
        out->kernels = L->n_ops;
        out->block = 1024;
        out->cluster = 1;
        out->grid = L->op_kind[0] == OP_GEMM_BF16 ? gemm_grid(L->op_gemm) : 16;
        out->smem = L->op_kind[0] == OP_GEMM_BF16 ? (int64_t)gemm_smem(L->op_gemm, false) : 0;
        out->param_bytes = (int64_t)sizeof(MkLaunch);
        return 0;
    }
    int kernels = 0;
    for (int i = 0; i < ST_COUNT; ++i) kernels += L->stage_on[i];
    if (L->use_segments || L->use_fused) kernels = 6 + (L->stage_on[ST_HROW] ? 1 : 0);  // attention x 2, A, g1, [h row], g2, B
    int64_t grid = 0, smem = 0;
    auto gg = [&](const GemmArgs& g, bool f32) {
        const int64_t n = gemm_grid(g);
        if (n > grid) grid = n;
        const int64_t sm = (int64_t)gemm_smem(g, f32);
        if (sm > smem) smem = sm;
    };
    if (L->is_head) {
        grid = (int64_t)(L->head_gemm.N / gemm_gws_bn(false)) * L->head_ks;
        smem = (int64_t)gemm_gws_smem(false, L->head_gemm.K, L->head_ks);
    } else {
        gg(L->oproj, false);
        gg(L->pooler, false);
        gg(L->router, true);
        gg(L->unpool, false);
        if (!L->shape.tail) gg(L->qkv, false);
    }
    const int64_t g1 = (int64_t)(L->ex.I_s / 16) * L->max_active, g2 = (int64_t)(L->ex.H_s / 16) * L->max_active;
    if (g1 > grid) grid = g1;
    if (g2 > grid) grid = g2;
    if ((int64_t)g1_smem(L->ex.P) > smem) smem = (int64_t)g1_smem(L->ex.P);
    if ((int64_t)g2_smem(L->ex.I) > smem) smem = (int64_t)g2_smem(L->ex.I);
    out->grid = grid;
    out->block = 1024;
    out->cluster = 1;
    out->smem = smem;
    out->kernels = kernels;
    out->param_bytes = (int64_t)sizeof(MkLaunch);
    return 0;
}

// ---- feeds, entry, lm_head, soft cap, accept ----

// the wait of the step's tail (soft cap or accept) for every rank's lm_head shard
static void logits_wait(XchgWait& w, uint64_t flags, int64_t contributors, int64_t budget, uint64_t status) {
    memset(&w, 0, sizeof w);
    if (flags == 0 || contributors <= 0) return;
    w.flag = (const unsigned*)flags + XP_LOGITS;
    w.epoch = (const unsigned*)flags + kXchgEpoch + XP_LOGITS;
    w.contributors = (unsigned)contributors;
    w.budget = budget > 0 ? budget : kDefaultWaitBudget;
    w.status = (int*)status;
    w.stage = 100 + XP_LOGITS;
}

static int lm_head_on_engine(MkModule* module, const MkLmHeadBind* b, MkLaunch** out);  // draft_host.inc

static MkLaunch* new_op_launch(MkModule* module, int kind) {
    MkLaunch* L = new (std::nothrow) MkLaunch();
    if (L == nullptr) return nullptr;
    L->pack_only = module == nullptr;
    L->device = module ? module->device : -1;
    L->sms = module ? module->sms : 148;
    L->n_ops = 1;
    L->op_kind[0] = kind;
    return L;
}

int mk_feeds_bind(MkModule* module, const MkFeedsBind* b, MkLaunch** out) {
    MK_REQUIRE(out != nullptr && b != nullptr, "bind or out is NULL");
    NEED(positions); NEED(out_cache_loc); NEED(seq_lens); NEED(req_pool_indices); NEED(req_to_token);
    NEED(loc_full); NEED(kv_len); NEED(pt_full);
    MK_REQUIRE(b->rows >= 1 && b->rows <= kMaxRows, "rows %lld outside 1..16", (long long)b->rows);
    MK_REQUIRE(b->r2t_rows >= 1 && b->r2t_width >= b->rows, "req_to_token is %lld x %lld", (long long)b->r2t_rows, (long long)b->r2t_width);
    MK_REQUIRE(b->cos_sin_cache == 0 || (b->cos_sin != 0 && b->cos_sin_rows > 0 && b->head_dim > 0), "rope cache without rows or output");
    MK_REQUIRE((b->swa_out_cache_loc == 0) == (b->loc_swa == 0), "swa_out_cache_loc and loc_swa go together");
    MK_REQUIRE((b->full_to_swa == 0) == (b->pt_swa == 0), "full_to_swa and pt_swa go together");
    MkLaunch* L = new_op_launch(module, OP_FEEDS);
    MK_REQUIRE(L != nullptr, "out of host memory");
    L->feeds = FeedsArgs{(const long long*)b->positions, (const float*)b->cos_sin_cache, b->cos_sin_rows, (const long long*)b->out_cache_loc,
                         (const long long*)b->swa_out_cache_loc, (const long long*)b->seq_lens, (const long long*)b->req_pool_indices,
                         (const int*)b->req_to_token, b->r2t_rows, b->r2t_width, (const long long*)b->full_to_swa, b->swa_map_len,
                         (float*)b->cos_sin, (int*)b->loc_full, (int*)b->loc_swa, (int*)b->kv_len, (long long*)b->pt_full,
                         (long long*)b->pt_swa, (int)b->rows, (int)b->head_dim, (int)b->kv_row_bytes, (int*)b->status};
    L->status = (int*)b->status;
    *out = L;
    return 0;
}

int mk_entry_bind(MkModule* module, const MkEntryBind* b, MkLaunch** out) {
    MK_REQUIRE(out != nullptr && b != nullptr, "bind or out is NULL");
    NEED(ids); NEED(pre_w); NEED(residual); NEED(normed);
    MK_REQUIRE(b->rows >= 1 && b->rows <= kMaxRows, "rows %lld outside 1..16", (long long)b->rows);
    MK_REQUIRE(b->hidden >= 256 && b->hidden <= 8192 && b->hidden % 256 == 0, "hidden %lld unsupported", (long long)b->hidden);
    MK_REQUIRE(b->ranks >= 1 && b->ranks <= MKH_RANKS && b->shard_rows >= 1, "ranks %lld / shard_rows %lld", (long long)b->ranks, (long long)b->shard_rows);
    MkLaunch* L = new_op_launch(module, OP_ENTRY);
    MK_REQUIRE(L != nullptr, "out of host memory");
    EntryArgs& e = L->entry;
    memset(&e, 0, sizeof e);
    e.ids = (const long long*)b->ids;
    for (int r = 0; r < b->ranks; ++r) {
        if (b->embed_peer[r] == 0 || (b->embed_peer[r] & 15)) {
            delete L;
            return fail("embed_peer[%d] is 0 or not 16-byte aligned", r);
        }
        e.embed[r] = (const bf16*)b->embed_peer[r];
    }
    e.shard_rows = b->shard_rows; e.ranks = (int)b->ranks; e.pre_w = (const bf16*)b->pre_w; e.residual = (float*)b->residual;
    e.normed = (bf16*)b->normed; e.rows = (int)b->rows; e.hidden = (int)b->hidden; e.eps_embed = (float)b->eps_embed; e.eps_pre = (float)b->eps_pre;
    *out = L;
    return 0;
}

int mk_lm_head_bind(MkModule* module, const MkLmHeadBind* b, MkLaunch** out) {
    MK_REQUIRE(out != nullptr && b != nullptr, "bind or out is NULL");
    NEED(w); NEED(x);
    ALIGNED16(w); ALIGNED16(x);
    MK_REQUIRE(b->rows >= 1 && b->rows <= kMaxRows, "rows %lld outside 1..16", (long long)b->rows);
    MK_REQUIRE(b->rank >= 0 && b->rank < MKH_RANKS && b->out_peer[b->rank] != 0, "out_peer[rank] (this rank's logits) is 0");
    MK_REQUIRE(b->n_out >= 1 && b->col0 >= 0 && b->col0 + b->n_out <= b->v_total, "columns [%lld, %lld) outside %lld", (long long)b->col0,
               (long long)(b->col0 + b->n_out), (long long)b->v_total);
    MK_REQUIRE(b->w_packed != 1 || (b->ws != 0 && b->hidden % 512 == 0), "w_packed 1 needs the item engine (ws and hidden a multiple of 512)");
    MK_REQUIRE(b->w_packed != 2 || (b->ws != 0 && b->hidden % 128 == 0), "w_packed 2 needs the tensor-core engine (ws and hidden a multiple of 128)");
    MK_REQUIRE(b->w_packed >= 0 && b->w_packed <= 2, "w_packed %lld is not 0, 1 or 2", (long long)b->w_packed);
    if (b->w_packed == 2 || (b->ws != 0 && b->hidden % 512 == 0)) return lm_head_on_engine(module, b, out);
    MkLaunch* L = new_op_launch(module, OP_GEMM_BF16);
    MK_REQUIRE(L != nullptr, "out of host memory");
    GemmArgs& g = L->op_gemm;
    memset(&g, 0, sizeof g);
    g.w = (const void*)b->w; g.x = (const void*)b->x;
    g.M = (int)b->rows; g.N = (int)b->n_out; g.K = (int)b->hidden; g.ldw = g.ldx = (int)b->hidden;
    if (gemm_plan(false, 0, g.N, g.K, L->sms, &g.wn, &g.ksplit)) {
        delete L;
        return fail("lm_head [%lld x %lld] has no tile / K-split plan", (long long)b->n_out, (long long)b->hidden);
    }
    for (int r = 0; r < MKH_RANKS; ++r)
        if (b->out_peer[r]) g.out[g.n_out++] = (void*)b->out_peer[r];
    g.ldo = (int)b->v_total; g.col0 = (int)b->col0; g.out_f32 = 1;
    g.status = L->status = (int*)b->status;
    if (b->flags) {
        unsigned* const flags = (unsigned*)b->flags;
        for (int r = 0; r < MKH_RANKS; ++r) {
            unsigned* f = (unsigned*)(r == b->rank ? b->flags : b->flags_peer[r]);
            if ((f != nullptr) != (b->out_peer[r] != 0)) {
                delete L;
                return fail("flags_peer[%d] and out_peer[%d] disagree on the rank's presence", r, r);
            }
            if (f) {
                g.sig.flag[g.sig.n++] = f + XP_LOGITS;
                g.sig.remote |= r != b->rank;
            }
        }
        g.sig.done = flags + kXchgDone + XP_LOGITS;
        g.sig.epoch = flags + kXchgEpoch + XP_LOGITS;
    }
    *out = L;
    return 0;
}

int mk_softcap_bind(MkModule* module, const MkSoftcapBind* b, MkLaunch** out) {
    MK_REQUIRE(out != nullptr && b != nullptr, "bind or out is NULL");
    NEED(x); NEED(out);
    MK_REQUIRE(b->numel >= 1 && b->cap > 0, "numel %lld / cap %g", (long long)b->numel, b->cap);
    MkLaunch* L = new_op_launch(module, OP_SOFTCAP);
    MK_REQUIRE(L != nullptr, "out of host memory");
    L->softcap = SoftcapArgs{(const float*)b->x, (float*)b->out, b->numel, (float)b->scale, (float)b->cap};
    logits_wait(L->softcap.wait, b->flags, b->contributors, b->wait_budget, b->status);
    L->status = (int*)b->status;
    *out = L;
    return 0;
}

int mk_accept_bind(MkModule* module, const MkAcceptBind* b, MkLaunch** out) {
    MK_REQUIRE(out != nullptr && b != nullptr, "bind or out is NULL");
    NEED(logits); NEED(tokens); NEED(words); NEED(out_ring); NEED(counter);
    MK_REQUIRE(b->samp != 0 || b->top1 != 0, "top1 is not bound");
    MK_REQUIRE(b->rows >= 1 && b->rows <= kMaxRows && b->b_live >= 1 && b->b_live <= b->rows, "rows %lld / b_live %lld", (long long)b->rows,
               (long long)b->b_live);
    MK_REQUIRE(b->vocab >= 1 && b->ring >= b->rows && b->cap > 0, "vocab %lld / ring %lld / cap %g", (long long)b->vocab, (long long)b->ring, b->cap);
    MK_REQUIRE(b->accept_override == 0 || b->n_override >= 1, "accept_override without entries");
    MK_REQUIRE(b->cos_sin == 0 || (b->cos_sin_cache != 0 && b->cos_sin_rows >= 1), "cos_sin without its cache");
    MK_REQUIRE(b->dslot == 0 || (b->dkv_len != 0 && b->dring >= 1), "dslot without dkv_len / dring");
    MK_REQUIRE(b->dcos_sin == 0 || (b->dslot != 0 && b->dcos_sin_cache != 0 && b->dcos_sin_rows >= 1), "dcos_sin without dslot or its cache");
    const int64_t cells = b->rows * b->vocab, ys_bytes = (cells * 4 + 255) / 256 * 256;
    if (b->samp != 0) {
        NEED(cand); NEED(walk_q); NEED(sample_ws);
        MK_REQUIRE(b->b_live >= 2, "the sampled accept needs at least one draft row");
        MK_REQUIRE(b->sample_ws_bytes >= ys_bytes + cells * 8 + 256, "sample_ws_bytes %lld below the %lld the sampled accept needs",
                   (long long)b->sample_ws_bytes, (long long)(ys_bytes + cells * 8 + 256));
        MK_REQUIRE((b->sample_ws & 255) == 0, "sample_ws is not 256-byte aligned");
    }
    MkLaunch* L = new_op_launch(module, OP_ACCEPT);
    MK_REQUIRE(L != nullptr, "out of host memory");
    L->accept = AcceptArgs{(const float*)b->logits, (int)b->vocab, (int)b->rows, (int)b->b_live, (float)b->scale, (float)b->cap,
                           (const long long*)b->tokens, (const int*)b->accept_override, (int)b->n_override, (long long*)b->words,
                           (int*)b->out_ring, (int)b->ring, (int*)b->top1, (unsigned*)b->counter, (const float*)b->cos_sin_cache,
                           b->cos_sin_rows, (float*)b->cos_sin, (int*)b->loc_full, (int*)b->loc_swa, (int*)b->kv_len,
                           (const float*)b->dcos_sin_cache, b->dcos_sin_rows, (float*)b->dcos_sin, (int*)b->dslot, (int*)b->dkv_len,
                           (int)b->dring};
    logits_wait(L->accept.wait, b->flags, b->contributors, b->wait_budget, b->status);
    L->accept.pool_rows = b->pool_rows;
    L->accept.status = (int*)b->status;
    if (b->samp != 0) {
        L->accept.samp = (const long long*)b->samp;
        L->accept.cand = (const long long*)b->cand;
        L->accept.walk_q = (const float*)b->walk_q;
        L->accept.block_verify = b->block_verify != 0;
        L->accept.ys = (float*)b->sample_ws;
        L->accept.es = (double*)(b->sample_ws + (uint64_t)ys_bytes);
        L->accept.row_z = (double*)(b->sample_ws + (uint64_t)ys_bytes + (uint64_t)cells * 8);
        L->accept.sample_out = (double*)b->sample_out;
    }
    MK_REQUIRE(b->tree == 0 || b->samp == 0, "the token tree's accept is greedy: samp and tree are exclusive");
    L->accept.tree = (int*)b->tree;
    L->status = (int*)b->status;
    *out = L;
    return 0;
}

// ---- layer 0's head ----

static int qkv_check(const MkQkvBind* b, MkQkvConstants* c) {
    MK_REQUIRE(b != nullptr, "bind is NULL");
    MK_REQUIRE(b->rows >= 1 && b->rows <= kMaxRows, "rows %lld outside 1..16", (long long)b->rows);
    MK_REQUIRE(b->q_heads >= 1 && b->kv_heads >= 1, "heads must be positive");
    MK_REQUIRE(b->hidden >= 256 && b->hidden <= 8192 && gemm_gws_ksplit(false, (int)b->hidden) > 0, "hidden %lld unsupported",
               (long long)b->hidden);
    c->qkv_row = 2 * (b->q_heads + b->kv_heads) * kHeadDim;
    c->kv_row_bytes = b->kv_heads * kHeadDim * 2;
    MK_REQUIRE(c->qkv_row / gemm_gws_bn(false) <= 1024, "qkv row %lld too wide", (long long)c->qkv_row);
    c->ws_bytes = (int64_t)align_up((size_t)16 * 16 * c->qkv_row * 4, 256) + 4096;
    c->kernels = 2;
    return 0;
}

// Fills the two argument records of the head from a bind and a scratch pointer (partials first, then the counters).
static int qkv_fill(const MkQkvBind* b, const MkQkvConstants& c, unsigned char* scratch, GemmGwsArgs& g, int& ks, RowopsArgs& r) {
    memset(&g, 0, sizeof g);
    g.w = (const void*)b->w;
    g.x = (const void*)b->x;
    g.M = (int)b->rows; g.N = (int)c.qkv_row; g.K = (int)b->hidden; g.ldw = g.ldx = (int)b->hidden;
    g.partial = (float*)scratch;
    g.counter = (unsigned*)(scratch + align_up((size_t)16 * 16 * c.qkv_row * 4, 256));
    g.out[0] = (void*)b->out;
    g.n_out = 1;
    g.ldo = (int)c.qkv_row;
    ks = gemm_gws_ksplit(false, g.K);
    MK_REQUIRE(ks > 0 && ks <= 16, "hidden %d has no supported K split", g.K);
    r = RowopsArgs{(bf16*)b->out, (const float*)b->cos_sin, (const int*)b->cache_loc, (unsigned char*)b->k_cache,
                   (unsigned char*)b->v_cache, (float)b->q_scale, (float)b->eps, (int)b->rows, (int)b->q_heads,
                   (int)b->kv_heads, (int)c.qkv_row, (int)c.kv_row_bytes};
    return 0;
}

int mk_qkv_constants(const MkQkvBind* bind, MkQkvConstants* out) {
    MK_REQUIRE(out != nullptr, "out is NULL");
    return qkv_check(bind, out);
}

int mk_qkv_bind(MkModule* module, const MkQkvBind* b, MkLaunch** out) {
    MK_REQUIRE(out != nullptr, "out is NULL");
    MkQkvConstants c;
    if (qkv_check(b, &c)) return -1;
    NEED(w); NEED(x); NEED(out); NEED(cache_loc); NEED(ws);
    ALIGNED16(w); ALIGNED16(x); ALIGNED16(out); ALIGNED16(ws);
    MK_REQUIRE((b->k_cache == 0) == (b->v_cache == 0), "k_cache and v_cache must be given together");
    MK_REQUIRE(b->ws_bytes >= c.ws_bytes, "ws_bytes %lld smaller than the %lld this shape needs", (long long)b->ws_bytes,
               (long long)c.ws_bytes);
    MkLaunch* L = new (std::nothrow) MkLaunch();
    MK_REQUIRE(L != nullptr, "out of host memory");
    L->pack_only = module == nullptr;
    L->device = module ? module->device : -1;
    memset(&L->shape, 0, sizeof L->shape);
    L->status = nullptr;
    for (int i = 0; i < ST_COUNT; ++i) L->stage_on[i] = false;
    L->stage_on[ST_QKV] = L->stage_on[ST_ROWOPS] = true;
    L->is_head = true;
    if (qkv_fill(b, c, (unsigned char*)b->ws, L->head_gemm, L->head_ks, L->rowops)) {
        delete L;
        return -1;
    }
    memset(&L->ex, 0, sizeof L->ex);
    L->max_active = 0;
    *out = L;
    return 0;
}

// ---- the head without any allocation: scratch inside the library's device image ----

// 16 K chunks x 16 rows x 4096 columns of f32 partial sums, then 1024 arrival counters.
static constexpr size_t kStaticPartialBytes = (size_t)16 * 16 * 4096 * 4;
static constexpr size_t kStaticCounterBytes = 4096;
static constexpr int64_t kStaticMaxQkvRow = 4096;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticPartialBytes + kStaticCounterBytes];
// On the host the array's name is only a handle for the runtime, not a device address: the address each device uses is
// looked up once with that device current and kept here.
static constexpr int kStaticMaxDevices = 64;
static unsigned char* g_static_addr[kStaticMaxDevices];
static std::mutex g_static_mutex;

static int static_scratch_for_current_device(unsigned char** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    MK_REQUIRE(dev >= 0 && dev < kStaticMaxDevices, "device ordinal %d beyond the %d this entry point tracks", dev, kStaticMaxDevices);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (g_static_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
        MK_REQUIRE(p != nullptr, "the static scratch has no address on device %d", dev);
        e = gemm_gws_prepare();
        if (e != cudaSuccess) return cuda_fail(e, "gemm_gws_prepare");
        g_static_addr[dev] = (unsigned char*)p;
    }
    *out = g_static_addr[dev];
    return 0;
}

int mk_qkv_launch_static(const MkQkvBind* b, uint64_t stream) {
    MkQkvConstants c;
    if (qkv_check(b, &c)) return -1;
    NEED(w); NEED(x); NEED(out); NEED(cache_loc);
    ALIGNED16(w); ALIGNED16(x); ALIGNED16(out);
    MK_REQUIRE((b->k_cache == 0) == (b->v_cache == 0), "k_cache and v_cache must be given together");
    MK_REQUIRE(c.qkv_row <= kStaticMaxQkvRow,
               "qkv row of %lld columns exceeds the %lld the built-in scratch holds: use mk_qkv_bind with caller scratch",
               (long long)c.qkv_row, (long long)kStaticMaxQkvRow);
    unsigned char* scratch = nullptr;
    if (static_scratch_for_current_device(&scratch)) return -1;
    GemmGwsArgs g;
    RowopsArgs r;
    int ks = 0;
    if (qkv_fill(b, c, scratch, g, ks, r)) return -1;
    MK_REQUIRE((unsigned char*)g.counter + kStaticCounterBytes <= scratch + sizeof g_static_scratch &&
                   (size_t)(g.N / gemm_gws_bn(false)) * 4 <= kStaticCounterBytes,
               "internal: counters outside the built-in scratch");
    // the array keeps whatever the previous call left: the arrival counters must start at zero (the partial sums are
    // fully overwritten before they are read)
    cudaError_t e = cudaMemsetAsync(g.counter, 0, kStaticCounterBytes, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(static counters)");
    e = gemm_gws_launch(g, false, ks, (cudaStream_t)stream, false);
    if (e != cudaSuccess) return cuda_fail(e, "qkv GEMM launch");
    e = rowops_launch(r, (cudaStream_t)stream, false);
    if (e != cudaSuccess) return cuda_fail(e, "qkv row ops launch");
    return 0;
}

// ---- memory shared between the ranks' processes ----

int mk_symm_alloc(int64_t bytes, uint64_t* ptr, unsigned char* handle) {
    MK_REQUIRE(ptr != nullptr && handle != nullptr, "ptr or handle is NULL");
    MK_REQUIRE(bytes > 0, "bytes %lld", (long long)bytes);
    static_assert(sizeof(cudaIpcMemHandle_t) <= MK_SYMM_HANDLE_BYTES, "handle does not fit");
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, (size_t)bytes);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc");
    e = cudaMemset(p, 0, (size_t)bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return cuda_fail(e, "cudaIpcGetMemHandle");
    }
    memset(handle, 0, MK_SYMM_HANDLE_BYTES);
    memcpy(handle, &h, sizeof h);
    *ptr = (uint64_t)p;
    return 0;
}

int mk_symm_open(const unsigned char* handle, uint64_t* ptr) {
    MK_REQUIRE(ptr != nullptr && handle != nullptr, "ptr or handle is NULL");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return cuda_fail(e, "cudaIpcOpenMemHandle");
    *ptr = (uint64_t)p;
    return 0;
}

int mk_symm_close(uint64_t ptr) {
    cudaError_t e = cudaIpcCloseMemHandle((void*)ptr);
    if (e != cudaSuccess) return cuda_fail(e, "cudaIpcCloseMemHandle");
    return 0;
}

int mk_symm_free(uint64_t ptr) {
    cudaError_t e = cudaFree((void*)ptr);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFree");
    return 0;
}

int mk_launch_status(const MkLaunch* launch, uint64_t stream, MkLaunchStatus* out) {
    MK_REQUIRE(launch != nullptr && out != nullptr, "launch or out is NULL");
    MK_REQUIRE(!launch->pack_only, "a pack-only record has no device status");
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
    int host[8] = {0};
    if (launch->status == nullptr) {
        memset(out, 0, sizeof *out);
        return 0;
    }
    e = cudaMemcpy(host, launch->status, sizeof host, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy(status)");
    out->code = host[0];
    out->stage = host[1];
    out->block = host[2];
    out->observed = host[3];
    out->expected = host[4];
    return 0;
}

}  // extern "C"

#include "draft_host.inc"
