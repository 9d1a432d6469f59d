// The dense GEMMs of the decode path (o_proj, pooler, router, unpooler, qkv head, lm_head, the draft's projections) on the
// 5th-generation tensor cores: out[m, n] = sum_k x[m, k] W[n, k] with at most 16 activation rows.
//
// Shape of the contraction ("swap-AB"): the WEIGHTS are the M = 128 operand of tcgen05.mma (kind::f16 for bf16 weights,
// kind::tf32 for the f32 router), the window's rows the N = 16 operand, the accumulator a [128 lanes x 16 columns] f32 block
// of tensor memory. The accumulation over K never leaves tensor memory while a CTA works on a tile.
//
// Work split ("stream-K"): a GEMM is tiles x K-stages stage units, a stage unit being 128 weight rows x 256 bytes of K
// (128 bf16 or 64 f32 elements: two 128-byte-swizzle atoms). The stage units of the launch's one or two GEMMs form one
// sequence that is cut into equal contiguous ranges, one per CTA, whatever the shape: every CTA streams the same number of
// bytes. A tile whose K range is shared by several CTAs is finished by the last of them to arrive: each writes its [16 x 128]
// f32 partial to L2-resident scratch, takes a ticket (atomicInc that wraps at the number of contributors, so the word is
// back at zero for the next launch), and the holder of the last ticket sums the partials in contributor order (a fixed
// order: results do not depend on timing) and runs the epilogue. There is no grid barrier and no second pass.
//
// Weight image (built once by the host, sgl_muse_mega_b200/muse_spark/b200/weights.py pack_umma): for every
// (tile, K stage) 32 KiB: atom 0 then atom 1, an atom = 128 rows x 128 bytes with the 16-byte chunk j of row r stored at
// chunk j ^ (r % 8) (the K-major 128-byte-swizzle operand layout); rows past N are zero. One stage arrives by two bulk
// copies (only the valid rows of a ragged last tile are read). The router's image has the low 13 mantissa bits cleared.
//
// Roles (256 threads): warp 0 lane 0 streams weight stages through a 6-deep ring (starting before the programmatic
// launch wait: weights do not depend on the predecessor), warps 2-3 copy the activation slice of every stage into the
// swizzled B layout with cp.async (three stages in flight per thread), warp 1 lane 0 issues the MMAs, warps 4-7 read the
// accumulators and run the epilogue (bf16 / f32 stores into every destination, router scores, the qkv row work, SwiGLU,
// the draft's conv and head work). Two accumulators alternate, so the MMAs of a CTA's next tile run under the epilogue
// of the previous one.
//
// The roles and the epilogues are device functions of dense.cuh (they keep their pipeline state from one GEMM stage to the
// next, so fused.cuh chains two stages and the row work between them in one kernel).
//
// Every wait is bounded: an expired wait raises the CTA's abort flag, records itself in the launch's status block (code 3)
// and every role leaves through the common teardown, which releases the tensor memory. Nothing traps.
//
// Reference counterparts: sm103/kernels/framework.cuh:349-706 (dense_body: kind::f16 tiles, TMEM accumulators, TMA ring,
// weights before griddepcontrol.wait), kernels/ptx.cuh:872-880 (kind::tf32 router).
#include "dense.cuh"

namespace mk {

namespace {
constexpr int kRing = 6;
}  // namespace


__global__ void __launch_bounds__(kDThreads, 1) dense_umma_kernel(const __grid_constant__ SegGemmArgs a) {
    extern __shared__ unsigned char dense_smem_raw[];
#ifdef DENSE_TRACE
    unsigned long long t_entry;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_entry));
#endif
    DenseCtx c = dense_setup_cta<kRing>(dense_smem_raw, a.status);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef DENSE_TRACE
    // o_proj 0, pooler + router 1, unpooler 2, qkv 3, anything else 4 + finish % 4
    c.trace_id = a.finish == 1 ? 1 : a.finish == 2 ? 3 : a.finish == 0 ? (a.g[0].K > 1024 ? 2 : 0) : 4 + (a.finish & 3);
    if (tid == 0) {
        g_dense_trace[c.trace_id][blockIdx.x][0] = t_entry;
        DT(1)
    }
#endif
    const Plan pl = plan_of(a);
    const TileSignals none = {{nullptr, nullptr}, {nullptr, nullptr}, false};
    if (warp == 0) {
        // weights do not depend on the predecessor: streamed before the programmatic launch wait
        if (lane == 0) {
            uint32_t it = 0;
            dense_produce<kRing>(a, c, pl, it, policy_evict_first());
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it = 0;
            int i = 0;
            dense_mma<kRing>(a, c, pl, it, i);
        }
    } else if (warp < 4) {
        griddep_wait();
        if (tid == 64) { DT(3) }
        uint32_t it = 0;
        dense_stage_x<kRing>(a, c, pl, it, tid - 64);
    } else {
        if (a.finish == 2 && tid - 128 < 33) {
            // the qkv head's rotation rows and pool slots (feeds of the step, written kernels ago): into L1 / L2 now, not at
            // the first tile's finish
            const char* p = tid - 128 < 32 ? (a.epi.cos_sin ? (const char*)a.epi.cos_sin + (tid - 128) * 128 : nullptr)
                                           : (const char*)a.epi.cache_loc;
            if (p != nullptr && (tid - 128 == 32 || (tid - 128) * 32 < a.g[0].M * 64)) asm volatile("prefetch.global.L1 [%0];" ::"l"(p));
        }
        griddep_wait();
        int i = 0;
        dense_epilogue<kRing>(a, c, pl, i, warp - 4, tid - 128, lane, none);
    }
    dense_teardown_cta(c);
    if (tid == 0) { DT(9) }
    xchg_signal(a.sig);
}

#ifdef DENSE_TRACE
}  // namespace mk
// trace builds: copies the dense launches' stamps to `dst` (8 x 160 x 16 words) and clears them
extern "C" int mk_dense_trace_read(void* dst) {
    if (cudaMemcpyFromSymbol(dst, mk::g_dense_trace, sizeof(unsigned long long) * 8 * 160 * 16) != cudaSuccess) return -1;
    static unsigned long long zero[8 * 160 * 16];
    return cudaMemcpyToSymbol(mk::g_dense_trace, zero, sizeof zero) == cudaSuccess ? 0 : -1;
}
namespace mk {
#endif

size_t dense_smem() { return DenseLayout<kRing>::kBytes; }

cudaError_t dense_prepare() {
    return cudaFuncSetAttribute(dense_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dense_smem());
}

static long long dense_units(const SegGemm& g) { return (long long)((g.N + 127) / 128) * (g.K * (g.f32 ? 4 : 2) / 256); }

int dense_grid(const SegGemmArgs& a, int sms) {
    long long T = dense_units(a.g[0]) + (a.n_gemm > 1 ? dense_units(a.g[1]) : 0);
    long long G = sms < kDenseMaxGrid ? sms : kDenseMaxGrid;
    if (T < G) G = T;
    return (int)(G < 1 ? 1 : G);
}

size_t dense_part_bound(long long N) { return (size_t)(2 * kDenseMaxGrid + 2 * ((N + 127) / 128)) * 2048; }

// Carves the launch's partial-sum scratch and tickets; false when they do not fit or a shape is not whole stages.
bool dense_setup(SegGemmArgs& a, int sms, float* part, size_t part_floats, unsigned* ticket, size_t ticket_words, int force_grid) {
    for (int i = 0; i < a.n_gemm; ++i) {
        const SegGemm& g = a.g[i];
        if (g.N < 1 || g.M < 1 || g.M > 16 || g.K < 1 || (g.K * (g.f32 ? 4 : 2)) % 256 != 0) return false;
        if (((uintptr_t)g.w & 15) || ((uintptr_t)g.x & 15) || (g.ldx & 15)) return false;
    }
    const long long T = dense_units(a.g[0]) + (a.n_gemm > 1 ? dense_units(a.g[1]) : 0);
    const int G = force_grid > 0 ? force_grid : dense_grid(a, sms);
    if (G > T) return false;  // every CTA owns at least one stage unit
    if (T * G >= (1ll << 31)) return false;  // the kernel cuts the units with 32-bit arithmetic
    const long long per = T / G;  // >= 1
    size_t used = 0, tickets = 0;
    for (int i = 0; i < a.n_gemm; ++i) {
        SegGemm& g = a.g[i];
        const long long KS = g.K * (g.f32 ? 4 : 2) / 256, tiles = (g.N + 127) / 128;
        g.maxc = (int)((KS + per - 1) / per + 1);
        g.part = part + used;
        g.ticket = ticket + tickets;
        used += (size_t)tiles * g.maxc * 2048;
        tickets += (size_t)tiles;
    }
    return used <= part_floats && tickets <= ticket_words;
}

cudaError_t dense_launch(const SegGemmArgs& a, int sms, cudaStream_t s, bool pdl) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(dense_grid(a, sms));
    cfg.blockDim = dim3(kDThreads);
    cfg.dynamicSmemBytes = dense_smem();
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, dense_umma_kernel, a);
}

}  // namespace mk
