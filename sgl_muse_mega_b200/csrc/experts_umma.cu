// The NVFP4 experts on the 5th-generation tensor cores: tcgen05.mma kind::mxf4nvf4.block_scale with the accumulators in
// tensor memory, weights streamed by 1-D bulk copies into a shared-memory ring, one persistent CTA per SM.
//
// Shapes ("swap-AB", as the contraction has at most 16 activation rows): the WEIGHTS are the M = 128 operand (A), the
// routed rows of the expert the N = 16 operand (B); K = 64 elements per instruction. A unit of work is (routed expert,
// block of 128 weight rows): g1 streams a PAIR of tiles per block (gate rows and the same up rows) so that the SwiGLU
// sees both halves of a feature in one thread; g2 streams one tile.
//
// Weight image (built once by the host packers, sgl_muse_mega_b200/muse_spark/b200/weights.py): for every
// (expert, block, K chunk of 256 elements) one contiguous stage
//     [tile 0: 128 rows x 128 B][tile 1 (g1 only)][scales tile 0: 4 x 512 B][scales tile 1]
// with the tiles already in the 128-byte-swizzle canonical layout and the scales in the 32 x 16 B image that
// tcgen05.cp.32x128b.warpx4 moves into tensor memory (byte n 16 + g 4 + k of a 512-B tile = scale of tile row 32 g + n,
// 16-element group k of that K64 block). One stage = 36 KiB (g1) or 18 KiB (g2) of bulk copies, no tensor map.
//
// Roles (256 threads): warp 0 lane 0 streams weight stages (full/empty mbarriers), warp 1 lane 0 copies the scales to
// tensor memory and issues the MMAs, warps 2-3 stage the routed rows two units ahead (codes into swizzled shared memory,
// their scale words and the unit's metadata beside them; warp 2 also owns the tensor-memory allocation), warps 4-7 move
// the staged scale words into tensor memory with tcgen05.st and run the epilogues from tensor memory:
// g1: gate/up -> bf16 -> SwiGLU -> per-16 requantisation of h -> the gathered planes of every peer;
// g2: x 2^e_row x alpha -> bf16 -> the gathered zb columns of every peer.
// Arithmetic contract: test/reference/muse_spark.py:438-563; reference kernels sm103/kernels/moe.cuh:1018-2458.
//
// Everything a unit needs besides its weights is fetched two units ahead, so that the rows of unit i + 2 are staged while
// unit i + 1 computes: two row tiles and two sets of row-scale words in shared memory, two accumulators in tensor memory.
// The row scales' place in tensor memory is single (256 columns: the block-scaled MMA wants a scale address on a
// 4-column boundary, so one K64 block takes 4 columns); it is refilled from shared memory in well under a microsecond once
// the previous unit's MMAs have completed. Measured before (everything staged after the previous unit): 5.4 us per unit
// with the weight ring full and the memory system idle, a third of the kernel.
//
// Tensor memory (512 columns): [0,64) two accumulator buffers of (gate 16 | up 16) columns, [64,96) weight scales of the
// stage in flight (4 columns per K64 block and tile), [128,384) row scales, one word per K64 block at a stride of 4.
// Every wait is bounded; an expired wait raises the CTA's abort flag, records itself in the status block and every role
// leaves through the common teardown, which releases the tensor memory.
#include "stages.h"
#include "umma.cuh"

namespace mk {

using namespace umma;

namespace {

constexpr uint32_t kTileBytes = 128 * 128;  // 128 rows x 256 e2m1
constexpr uint32_t kSfBytes = 4 * 512;      // 4 K64 blocks x (128 rows x 4 bytes)
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColAcc = 0, kColSfa = 64, kColSfb = 128;
constexpr int kMaxKChunks = 16;  // K <= 4096
constexpr uint32_t kXsBytes = kMaxKChunks * 2048;

struct UnitMeta {
    int n_tok, expert;
    int row[kMaxRows];    // source row of the B operand (token for g1, slot for g2)
    int slot[kMaxRows];   // route slot (token x topk + k)
    float s[kMaxRows];    // g1: alpha x x_scale[token]; g2: 2^e_row[slot]
    float c;              // g1: scale_c; g2: alpha
    int erow[kMaxRows];   // g2 without an h-row kernel: each routed slot's row exponent (the largest of its group exponents)
};

__device__ __forceinline__ void record_abort(int* status, volatile int* abort, int code, int where, int observed) {
    if (atomicExch((int*)abort, 1) == 0 && status != nullptr) {
        status[1] = where;
        status[2] = (int)blockIdx.x;
        status[3] = observed;
        status[4] = 0;
        __threadfence();
        status[0] = code;
    }
}

__device__ __forceinline__ int prov_exp_u(float amax) {
    const int b = __float_as_int(amax);
    const int bump = ((b & 0x7FFFFF) > 0x280000) || (b > 0x7F800000);
    return max((b >> 23) - 138 + bump, -120);
}

}  // namespace

// Trace builds (-DUMMA_TRACE): CTA 0 stamps the global timer into words [64 + 128 G2, ...) of the status block, four per
// unit: operands ready (MMA thread), last stage issued (MMA thread), accumulators complete (epilogue), next unit's row
// scales published (epilogue). Measured on the full shape: 14.0 us (g1) / 6.5 us (g2) from ready to issued, i.e. the weight
// stream at the SM's share of HBM bandwidth, then 1.5 us until the next unit is ready.
#ifdef UMMA_TRACE
#define UT(slot)                                                                                  \
    if (blockIdx.x == 0 && a.status != nullptr && (slot) < 60) {                                  \
        unsigned long long t_;                                                                    \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                    \
        ((unsigned long long*)(a.status + 64 + 128 * G2))[(slot)] = t_;                           \
    }
// and every CTA stamps its own milestones (16 words each) into a device array: 0 entry, 1 set up, 2 tables copied,
// 3 last weight stage issued, 4 first operands ready, 5 first weight stage landed, 6 last MMA committed, 7 first
// accumulators complete, 8 epilogues done, 9 torn down, 11 first rows staged
static __device__ unsigned long long g_umma_trace[2][160][16];
#define CT(slot)                                                       \
    {                                                                  \
        unsigned long long t_;                                         \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));         \
        g_umma_trace[G2][blockIdx.x][(slot)] = t_;                     \
    }
#else
#define UT(slot)
#define CT(slot)
#endif

template <bool G2>
__global__ void __launch_bounds__(256, 1) experts_umma_kernel(const UmmaArgs a) {
    constexpr int TILES = G2 ? 1 : 2;
    constexpr uint32_t STAGE = TILES * (kTileBytes + kSfBytes);
    constexpr int S = G2 ? 8 : 4;
    constexpr uint32_t IDESC = idesc_nvf4(128, 16);

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* stages = smem;
    unsigned char* xs = smem + S * STAGE;                   // 2 buffers of K/256 chunks of [16 rows x 128 B], swizzled
    uint32_t* sfw = (uint32_t*)(xs + 2 * kXsBytes);         // 2 x [16 rows][64] row-scale words (4 e4m3 per K64 block)
    UnitMeta* meta = (UnitMeta*)(sfw + 2 * kMaxRows * 64);  // two units in flight
    RouteTables* rt = (RouteTables*)(meta + 2);             // the launch's route tables, copied once
    uint64_t* bars = (uint64_t*)(((uintptr_t)(rt + 1) + 15) & ~(uintptr_t)15);
    uint64_t* full = bars;
    uint64_t* empty = bars + S;
    uint64_t* x_ready = bars + 2 * S;        // [2]
    uint64_t* acc_full = bars + 2 * S + 2;   // [2]
    uint64_t* acc_empty = bars + 2 * S + 4;  // [2]
    uint64_t* staged = bars + 2 * S + 6;     // [2] stager -> epilogue warps: rows, words and metadata of a unit are in place
    uint64_t* buf_free = bars + 2 * S + 8;   // [2] epilogue warps -> stager: the unit that used the buffer is finished
    uint64_t* rows_first = bars + 2 * S + 10;  // stager -> producer (g1): the first unit's row loads are on their way
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * S + 11);
    volatile int* abort = (volatile int*)(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        CT(0)
        for (int i = 0; i < S; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&x_ready[i], 128);
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 128);
            mbar_init(&staged[i], 64);
            mbar_init(&buf_free[i], 128);
        }
        mbar_init(rows_first, 64);
        *abort = 0;
        mbar_fence_init();
    }
    if (warp == 2) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    if (tid == 0) { CT(1) }

    // One round trip for the route tables every unit looks up. g2's predecessor is g1: the tables were written two or more
    // kernels back, so g2 copies them and starts streaming its first weights under g1's tail; the roles that touch what g1
    // wrote wait below.
    if (!G2) {
        griddep_wait_only();
        if (a.sig.target != nullptr && blockIdx.x == 0) {  // g2 will not wait for this grid's end: leave it the epoch to wait for
            if (tid == 0) xchg_announce(a.sig);
            __syncthreads();
        }
        griddep_launch();
    }
    for (int i = tid; i < (int)(sizeof(RouteTables) / 4); i += 256) ((int*)rt)[i] = ((const int*)a.rt)[i];
    __syncthreads();
    const int NB = a.NB, KCH = a.K / 256;
    const int n_units = rt->n_active * NB;
    if (tid == 0) { CT(2) }

    if (warp == 0) {
        // ---- weight producer ----
        if (lane == 0) {
            const uint64_t policy = policy_evict_first();  // expert weights are read once a step
            uint32_t it = 0;
            // g1 starts everything at once behind the routing kernel: the first unit's rows (32 KB) are requested before the
            // weight stream fills the memory system's queues with 21 MB, or they arrive behind it (4 us instead of 1)
            if (!G2 && blockIdx.x < n_units) mbar_wait(rows_first, 0, abort);
            for (int u = blockIdx.x; u < n_units && !*abort; u += gridDim.x) {
                const int e = rt->act_e[u / NB], blk = u % NB;
                const unsigned char* src = a.wpack + ((size_t)(e * NB + blk) * KCH) * STAGE;
                for (int kc = 0; kc < KCH; ++kc, ++it) {
                    const uint32_t s = it % S, round = it / S;
                    if (!mbar_wait(&empty[s], (round & 1) ^ 1, abort)) {
                        record_abort(a.status, abort, 3, 100 + G2, (int)it);
                        break;
                    }
                    mbar_arrive_expect_tx(&full[s], STAGE);
                    unsigned char* dst = stages + s * STAGE;
                    const unsigned char* g = src + (size_t)kc * STAGE;
#pragma unroll
                    for (uint32_t off = 0; off < STAGE; off += 9216) bulk_g2s_hint(dst + off, g + off, 9216, &full[s], policy);
                }
            }
            CT(3)
        }
    } else if (warp == 1) {
        // ---- scale copies + MMA issue ----
        if (lane == 0) {
            uint32_t it = 0;
            int i = 0;
            for (int u = blockIdx.x; u < n_units && !*abort; u += gridDim.x, ++i) {
                const int buf = i & 1;
                const uint32_t ph = (i >> 1) & 1;
                if (!mbar_wait(&x_ready[buf], ph, abort) || !mbar_wait(&acc_empty[buf], ph ^ 1, abort)) {
                    record_abort(a.status, abort, 3, 110 + G2, i);
                    break;
                }
                tc_fence_after();
                UT(4 * i + 0)
                if (i == 0) { CT(4) }
                const uint32_t xs_addr = smem_u32(xs + buf * kXsBytes);
                bool ok = true;
                for (int kc = 0; kc < KCH; ++kc, ++it) {
                    const uint32_t s = it % S, round = it / S;
                    if (!mbar_wait(&full[s], round & 1, abort)) {
                        record_abort(a.status, abort, 3, 120 + G2, (int)it);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    if (it == 0) { CT(5) }
                    const uint32_t sbase = smem_u32(stages + s * STAGE);
#pragma unroll
                    for (int t = 0; t < TILES; ++t)
#pragma unroll
                        for (int kb = 0; kb < 4; ++kb)
                            cp_sf(tmem + kColSfa + (t * 4 + kb) * 4, desc_sf(sbase + TILES * kTileBytes + t * kSfBytes + kb * 512));
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        const uint64_t bdesc = desc_sw128(xs_addr + kc * 2048 + kb * 32);
                        const uint32_t sfb = tmem + kColSfb + (kc * 4 + kb) * 4;
#pragma unroll
                        for (int t = 0; t < TILES; ++t)
                            mma_nvf4(tmem + kColAcc + buf * 32 + t * 16, desc_sw128(sbase + t * kTileBytes + kb * 32), bdesc, IDESC,
                                     tmem + kColSfa + (t * 4 + kb) * 4, sfb, (kc | kb) != 0);
                    }
                    tc_commit(&empty[s]);
                }
                if (!ok) break;
                UT(4 * i + 1)
                tc_commit(&acc_full[buf]);
                CT(6)
            }
        }
    } else if (warp < 4) {
        // ---- stager: the B operand of unit j into buffer j & 1, two units ahead of the MMAs ----
        const int ts = tid - 64;  // 0..63
        if (G2) {
            // a.wait.packets: the h planes' counter word counts this rank's own g1 too, so it alone orders the stager
            // behind g1's stores (its loads of the planes go through L2): no wait for g1's grid to end
            if (a.wait.packets) griddep_launch();
            else griddep_wait();
            xchg_wait_role(a.wait, ts, 64, 3);  // without an h-row kernel in front: every rank's column band of the h planes
        }
        int j = 0;
        for (int u = blockIdx.x; u < n_units; u += gridDim.x, ++j) {
            const int buf = j & 1;
            bool ok = j < 2 || mbar_wait(&buf_free[buf], ((j - 2) >> 1) & 1, abort);
            ok = bar_all(3, 64, ok);
            if (!ok) {
                if (ts == 0) record_abort(a.status, abort, 3, 140 + G2, j);
                break;
            }
            UnitMeta& m = meta[buf];
            unsigned char* xb = xs + buf * kXsBytes;
            uint32_t* wb = sfw + buf * (kMaxRows * 64);
            const int ai = u / NB, s0 = rt->act_off[ai], n_tok = rt->act_off[ai + 1] - s0, e = rt->act_e[ai];
            const int row_bytes = a.K / 2, per_row = KCH * 8, total = n_tok * per_row, wq = KCH, wtotal = n_tok * wq;
            // the rows' codes go straight to their swizzled places (16-byte asynchronous copies, all in flight at once);
            // every other global load of the unit is issued before the first store: one memory round trip
            for (int idx = ts; idx < total; idx += 64) {
                const int tk = idx / per_row, rem = idx - tk * per_row, kc = rem >> 3, jj = rem & 7;
                const int sl = rt->slot[s0 + tk];
                // only live rows are written: a stale row feeds accumulator columns that no epilogue reads
                cp_async16(xb + kc * 2048 + (tk >> 3) * 1024 + (tk & 7) * 128 + ((jj ^ (tk & 7)) << 4),
                           a.bq + (size_t)(G2 ? sl : sl / a.topk) * row_bytes + rem * 16, true);
            }
            cp_async_commit();
            int slot = 0, row = 0;
            float sc = 0.f, cc = 0.f;
            if (ts < n_tok) {
                slot = rt->slot[s0 + ts];
                row = G2 ? slot : slot / a.topk;
                sc = G2 ? (a.bex != nullptr ? 0.f : a.rowscale[slot]) : a.g1_alphas[e] * a.x_scale[row];
            }
            if (ts == 0) cc = G2 ? a.g2_alphas[e] : a.g1_scale_c[e];
            const bool view = G2 && a.bex != nullptr;  // this kernel forms the h-row view itself (no h-row kernel ran)
            uint4 wv[4], xv[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int idx = k * 64 + ts;  // 16 rows x 16 uint4 at most
                if (idx < wtotal) {
                    const int tk = idx / wq, c = idx - tk * wq;
                    const int sl = rt->slot[s0 + tk];
                    wv[k] = __ldcg((const uint4*)(a.bsf + (size_t)(G2 ? sl : sl / a.topk) * (a.K / 16) + c * 16));
                    if (view) xv[k] = __ldcg((const uint4*)(a.bex + (size_t)sl * (a.K / 16) + c * 16));
                }
            }
            if (j == 0) mbar_arrive(rows_first);  // the first unit's loads are issued: the weight stream may start (g1)
            if (view) {
                // the row exponent of each routed slot = the largest of its K / 16 group exponents: four threads share a
                // slot (a quarter of its exponent bytes each; tokens 0..7 on the first stager warp, 8..15 on the second)
                const int tk = ts >> 2, qd = ts & 3, gb = a.K / 16;
                int er = -128;
                if (tk < n_tok) {
                    const signed char* ex = a.bex + (size_t)rt->slot[s0 + tk] * gb;
                    uint4 v4[kMaxKChunks / 4];  // K <= 4096: at most 256 exponent bytes a slot, 64 a thread, loaded at once
#pragma unroll
                    for (int r = 0; r < kMaxKChunks / 4; ++r) {
                        const int i = qd * 16 + r * 64;
                        v4[r] = i < gb ? __ldcg((const uint4*)(ex + i)) : make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);
                    }
#pragma unroll
                    for (int r = 0; r < kMaxKChunks / 4; ++r) {
                        const uint32_t w4[4] = {v4[r].x, v4[r].y, v4[r].z, v4[r].w};
#pragma unroll
                        for (int j = 0; j < 4; ++j)
#pragma unroll
                            for (int b = 0; b < 4; ++b) er = max(er, (int)(signed char)(w4[j] >> (8 * b)));
                    }
                }
                er = max(er, __shfl_xor_sync(0xffffffffu, er, 1));
                er = max(er, __shfl_xor_sync(0xffffffffu, er, 2));
                if (qd == 0 && tk < n_tok) m.erow[tk] = er;
                bar_sync(3, 64);
                if (ts < n_tok) sc = __uint_as_float((uint32_t)(m.erow[ts] + 127) << 23);  // 2^e_row
                // every scale byte moved to its row's exponent (scale x 2^-(e_row - e_group))
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int idx = k * 64 + ts;
                    if (idx < wtotal) {
                        const int e_row = m.erow[idx / wq];
                        const uint32_t sw[4] = {wv[k].x, wv[k].y, wv[k].z, wv[k].w};
                        const uint32_t ew[4] = {xv[k].x, xv[k].y, xv[k].z, xv[k].w};
                        uint32_t o[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            o[j] = 0;
#pragma unroll
                            for (int b = 0; b < 4; ++b)
                                o[j] |= scale_down_byte((sw[j] >> (8 * b)) & 0xFFu, e_row - (int)(signed char)(ew[j] >> (8 * b))) << (8 * b);
                        }
                        wv[k] = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int idx = k * 64 + ts;
                if (idx < wtotal) {
                    const int tk = idx / wq, c = idx - tk * wq;
                    *(uint4*)(wb + tk * 64 + c * 4) = wv[k];
                }
            }
            if (ts < kMaxRows) {
                m.slot[ts] = slot;
                m.row[ts] = row;
                m.s[ts] = sc;
                if (ts == 0) {
                    m.n_tok = n_tok;
                    m.expert = e;
                    m.c = cc;
                }
            }
            cp_async_wait<0>();
            fence_proxy_async_smem();
            mbar_arrive(&staged[buf]);
            if (j == 0 && ts == 0) { CT(11) }
        }
    } else {
        // ---- scale words -> tensor memory, epilogue out ----
        if (G2) {  // nothing here reads what g1 wrote (the stager hands the rows over through shared memory)
            if (a.wait.packets) griddep_launch();
            else griddep_wait();
        }
        const int q = warp - 4, te = tid - 128;
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;

        // Unit i's row scales from shared to tensor memory (lane l = row l, the word of K64 block b at column 4 b; every
        // epilogue warp fills its own 32-lane quadrant), then the unit's B operand is handed to the MMA thread. Called once
        // the MMAs of unit i - 1 have completed: they were the last readers of these columns. Returns false on a timeout.
        auto publish = [&](int i) -> bool {
            const int buf = i & 1;
            if (!bar_all(2, 128, mbar_wait(&staged[buf], (i >> 1) & 1, abort))) return false;
            const uint32_t* src = sfw + buf * (kMaxRows * 64) + (lane & 15) * 64;
            for (int c = 0; c < KCH; ++c) {
                const uint4 w = *(const uint4*)(src + c * 4);
                const uint32_t r[16] = {w.x, 0, 0, 0, w.y, 0, 0, 0, w.z, 0, 0, 0, w.w, 0, 0, 0};
                tmem_st16(tmem + lane_base + kColSfb + c * 16, r);
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&x_ready[buf]);
            return true;
        };

        const int u0 = blockIdx.x, stride = gridDim.x;
        bool alive = u0 >= n_units || publish(0);
        int i = 0;
        for (int u = u0; alive && u < n_units; u += stride, ++i) {
            const int buf = i & 1;
            // all 128 epilogue threads agree on the outcome of a wait before any of them meets the others at a barrier again
            if (!bar_all(2, 128, mbar_wait(&acc_full[buf], (i >> 1) & 1, abort))) break;
            tc_fence_after();
            if (te == 0) { UT(4 * i + 2) }
            if (te == 0 && i == 0) { CT(7) }
            if (u + stride < n_units && !publish(i + 1)) break;
            if (te == 0) { UT(4 * i + 3) }
            const UnitMeta& m = meta[buf];
            const int blk = u % NB, n_tok = m.n_tok;
            const int mrow = q * 32 + lane;  // weight row of this thread inside the block
            if (!G2) {
                uint32_t rg[16], ru[16];
                tmem_ld16(tmem + lane_base + kColAcc + buf * 32, rg);
                tmem_ld16(tmem + lane_base + kColAcc + buf * 32 + 16, ru);
                tmem_ld_wait();
                // a quantisation group is 16 consecutive features = 16 consecutive lanes: the group's maximum and its
                // packed codes are formed with shuffles inside each half warp, one routed row at a time
#pragma unroll
                for (int t = 0; t < kMaxRows; ++t) {
                    if (t < n_tok) {
                        const float a1 = m.s[t];
                        const float g = bf16_round(__uint_as_float(rg[t]) * a1), up = bf16_round(__uint_as_float(ru[t]) * a1);
                        const float z = ((g / (1.0f + expf(-g))) * up) * m.c;
                        float amax = fabsf(z);
#pragma unroll
                        for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                        const int eg = prov_exp_u(amax);
                        const float down = __uint_as_float((uint32_t)(127 - eg) << 23);
                        const uint32_t sfb = float_to_e4m3((amax * down) * (1.0f / 6.0f));
                        const float d = e4m3_to_float(sfb);
                        const float inv = d > 0.f ? 1.0f / d : 0.f;
                        uint32_t word = float_to_e2m1((z * down) * inv) << (4 * (lane & 7));
#pragma unroll
                        for (int o = 4; o > 0; o >>= 1) word |= __shfl_xor_sync(0xffffffffu, word, o);
                        const uint32_t other = __shfl_xor_sync(0xffffffffu, word, 8);
                        if ((lane & 15) == 0) {
                            const int slot = m.slot[t], gcol = (a.rank * a.I_s + blk * 128) / 16 + (mrow >> 4);
                            for (int p = 0; p < a.n_peer; ++p) {
                                *(uint2*)(a.z_peer[p] + (size_t)slot * (a.I / 2) + gcol * 8) = make_uint2(word, other);
                                a.zsf_peer[p][(size_t)slot * (a.I / 16) + gcol] = (unsigned char)sfb;
                                a.zex_peer[p][(size_t)slot * (a.I / 16) + gcol] = (signed char)eg;
                            }
                        }
                    }
                }
            } else {
                uint32_t r[16];
                tmem_ld16(tmem + lane_base + kColAcc + buf * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int t = 0; t < kMaxRows; ++t) {
                    if (t < n_tok) {
                        const bf16 v = __float2bfloat16_rn((__uint_as_float(r[t]) * m.s[t]) * m.c);
                        const size_t off = (size_t)m.slot[t] * a.P + a.rank * a.H_s + blk * 128 + mrow;
                        for (int p = 0; p < a.n_peer; ++p) a.zb_peer[p][off] = v;
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&acc_empty[buf]);
            mbar_arrive(&buf_free[buf]);
        }
        if (te == 0 && *abort == 0 && i * stride + u0 < n_units) record_abort(a.status, abort, 3, 130 + G2, i);
        if (te == 0) { CT(8) }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2) tmem_dealloc(tmem, kTmemCols);
    if (tid == 0) { CT(9) }
    xchg_signal(a.sig);  // every CTA arrives, also one that had no unit
}

size_t experts_umma_smem(bool g2) {
    const size_t stage = (g2 ? 1 : 2) * (size_t)(kTileBytes + kSfBytes);
    const int S = g2 ? 8 : 4;
    return 1024 + S * stage + 2 * kXsBytes + 2 * kMaxRows * 64 * 4 + 2 * sizeof(UnitMeta) + sizeof(RouteTables) + 16 +
           (2 * S + 11) * 8 + 16;
}

cudaError_t experts_umma_prepare() {
    cudaError_t e = cudaFuncSetAttribute(experts_umma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)experts_umma_smem(false));
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(experts_umma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)experts_umma_smem(true));
}

#ifdef UMMA_TRACE
}  // namespace mk
// trace builds: copies the experts' per-CTA stamps to `dst` (2 x 160 x 16 words)
extern "C" int mk_umma_trace_read(void* dst) {
    return cudaMemcpyFromSymbol(dst, mk::g_umma_trace, sizeof(unsigned long long) * 2 * 160 * 16) == cudaSuccess ? 0 : -1;
}
namespace mk {
#endif

cudaError_t experts_umma_launch(const UmmaArgs& a, bool g2, int grid, cudaStream_t s, bool pdl) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = experts_umma_smem(g2);
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return g2 ? cudaLaunchKernelEx(&cfg, experts_umma_kernel<true>, a) : cudaLaunchKernelEx(&cfg, experts_umma_kernel<false>, a);
}

}  // namespace mk
