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
// 16-element group k of that K64 block). One stage = one bulk copy = 36 KiB (g1) or 18 KiB (g2), no tensor map.
//
// Roles (256 threads): warp 0 lane 0 streams weight stages (full/empty mbarriers), warp 1 lane 0 copies the scales to
// tensor memory and issues the MMAs, warp 2 owns the tensor-memory allocation, warps 4-7 stage the routed rows (codes
// into swizzled shared memory, their scales into tensor memory with tcgen05.st) and run the epilogues from tensor memory:
// g1: gate/up -> bf16 -> SwiGLU -> per-16 requantisation of h -> the gathered planes of every peer;
// g2: x 2^e_row x alpha -> bf16 -> the gathered zb columns of every peer.
// Arithmetic contract: test/reference/muse_spark.py:438-563; reference kernels sm103/kernels/moe.cuh:1018-2458.
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

struct UnitMeta {
    int n_tok, expert;
    int row[kMaxRows];    // source row of the B operand (token for g1, slot for g2)
    int slot[kMaxRows];   // route slot (token x topk + k)
    float s[kMaxRows];    // g1: alpha x x_scale[token]; g2: 2^e_row[slot]
    float c;              // g1: scale_c; g2: alpha
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

template <bool G2>
__global__ void __launch_bounds__(256, 1) experts_umma_kernel(const UmmaArgs a) {
    constexpr int TILES = G2 ? 1 : 2;
    constexpr uint32_t STAGE = TILES * (kTileBytes + kSfBytes);
    constexpr int S = G2 ? 10 : 5;
    constexpr uint32_t IDESC = idesc_nvf4(128, 16);

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* stages = smem;
    unsigned char* xs = smem + S * STAGE;                   // K/256 chunks of [16 rows x 128 B], swizzled
    float* zs = (float*)(xs + kMaxKChunks * 2048);          // g1: [16 rows][129] transpose buffer
    UnitMeta* meta = (UnitMeta*)(zs + 16 * 129 + 1);        // two units in flight
    uint64_t* bars = (uint64_t*)(((uintptr_t)(meta + 2) + 15) & ~(uintptr_t)15);
    uint64_t* full = bars;
    uint64_t* empty = bars + S;
    uint64_t* x_ready = bars + 2 * S;
    uint64_t* acc_full = bars + 2 * S + 1;
    uint64_t* acc_empty = bars + 2 * S + 3;
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * S + 5);
    volatile int* abort = (volatile int*)(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < S; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        mbar_init(x_ready, 128);
        mbar_init(&acc_full[0], 1);
        mbar_init(&acc_full[1], 1);
        mbar_init(&acc_empty[0], 128);
        mbar_init(&acc_empty[1], 128);
        *abort = 0;
        mbar_fence_init();
    }
    if (warp == 2) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    griddep_wait();
    const RouteTables* rt = a.rt;
    const int NB = a.NB, KCH = a.K / 256;
    const int n_units = rt->n_active * NB;

    if (warp == 0) {
        // ---- weight producer ----
        if (lane == 0) {
            uint32_t it = 0;
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
                    for (uint32_t off = 0; off < STAGE; off += 9216) bulk_g2s(dst + off, g + off, 9216, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ---- scale copies + MMA issue ----
        if (lane == 0) {
            uint32_t it = 0;
            int i = 0;
            for (int u = blockIdx.x; u < n_units && !*abort; u += gridDim.x, ++i) {
                const int buf = i & 1;
                if (!mbar_wait(x_ready, i & 1, abort) || !mbar_wait(&acc_empty[buf], ((i >> 1) & 1) ^ 1, abort)) {
                    record_abort(a.status, abort, 3, 110 + G2, i);
                    break;
                }
                tc_fence_after();
                const uint32_t xs_addr = smem_u32(xs);
                bool ok = true;
                for (int kc = 0; kc < KCH; ++kc, ++it) {
                    const uint32_t s = it % S, round = it / S;
                    if (!mbar_wait(&full[s], round & 1, abort)) {
                        record_abort(a.status, abort, 3, 120 + G2, (int)it);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
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
                tc_commit(&acc_full[buf]);
            }
        }
    } else if (warp >= 4) {
        // ---- routed rows in, epilogue out ----
        const int q = warp - 4, te = tid - 128;
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;

        auto load_b = [&](int u, int i) {
            UnitMeta& m = meta[i & 1];
            const int ai = u / NB, s0 = rt->act_off[ai], n_tok = rt->act_off[ai + 1] - s0, e = rt->act_e[ai];
            if (te < kMaxRows) {
                int slot = 0, row = 0;
                float sc = 0.f;
                if (te < n_tok) {
                    slot = rt->slot[s0 + te];
                    row = G2 ? slot : slot / a.topk;
                    sc = G2 ? a.rowscale[slot] : a.g1_alphas[e] * a.x_scale[row];
                }
                m.slot[te] = slot;
                m.row[te] = row;
                m.s[te] = sc;
                if (te == 0) {
                    m.n_tok = n_tok;
                    m.expert = e;
                    m.c = G2 ? a.g2_alphas[e] : a.g1_scale_c[e];
                }
            }
            bar_sync(1, 128);
            // codes -> swizzled K-major tile rows. Only the n_tok live rows are written: a stale row only feeds accumulator
            // columns that no epilogue reads (the columns of an MMA are independent). All loads of a batch are issued
            // before the first store, so a batch costs one memory round trip, not one per chunk.
            const int row_bytes = a.K / 2, per_row = KCH * 8, total = n_tok * per_row;
            for (int base = 0; base < total; base += 128 * 8) {
                uint4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int idx = base + u * 128 + te;
                    if (idx < total) {
                        const int tk = idx / per_row, rem = idx - tk * per_row;
                        v[u] = *(const uint4*)(a.bq + (size_t)m.row[tk] * row_bytes + rem * 16);
                    }
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int idx = base + u * 128 + te;
                    if (idx < total) {
                        const int tk = idx / per_row, rem = idx - tk * per_row, kc = rem >> 3, j = rem & 7;
                        *(uint4*)(xs + kc * 2048 + (tk >> 3) * 1024 + (tk & 7) * 128 + ((j ^ (tk & 7)) << 4)) = v[u];
                    }
                }
            }
            // row scales -> tensor memory: lane l = row l, one word (4 e4m3) per K64 block at a column stride of 4;
            // every epilogue warp writes its own 32-lane quadrant with the same words. The row's words are fetched in one
            // batch of 16-byte loads, then stored 16 columns at a time.
            const bool live = lane < n_tok;
            const uint32_t* sfrow = (const uint32_t*)(a.bsf + (size_t)(live ? m.row[lane] : 0) * (a.K / 16));
            uint4 w[kMaxKChunks];
#pragma unroll
            for (int c = 0; c < kMaxKChunks; ++c) w[c] = (live && c < KCH) ? *(const uint4*)(sfrow + c * 4) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int c = 0; c < kMaxKChunks; ++c) {
                if (c < KCH) {
                    uint32_t r[16];
#pragma unroll
                    for (int k = 0; k < 16; ++k) r[k] = 0;
                    r[0] = w[c].x;
                    r[4] = w[c].y;
                    r[8] = w[c].z;
                    r[12] = w[c].w;
                    tmem_st16(tmem + lane_base + kColSfb + c * 16, r);
                }
            }
            tmem_st_wait();
            tc_fence_before();
            fence_proxy_async_smem();
            mbar_arrive(x_ready);
        };

        int i = 0;
        if ((int)blockIdx.x < n_units) load_b(blockIdx.x, 0);
        for (int u = blockIdx.x; u < n_units; u += gridDim.x, ++i) {
            const int buf = i & 1;
            // all 128 epilogue threads agree on the outcome before any of them meets the others at a barrier again
            const bool ok = bar_all(2, 128, mbar_wait(&acc_full[buf], (i >> 1) & 1, abort));
            if (!ok) {
                if (te == 0) record_abort(a.status, abort, 3, 130 + G2, i);
                break;
            }
            tc_fence_after();
            if (u + (int)gridDim.x < n_units) load_b(u + gridDim.x, i + 1);
            const UnitMeta& m = meta[buf];
            const int blk = u % NB, n_tok = m.n_tok;
            const int mrow = q * 32 + lane;  // weight row of this thread inside the block
            if (!G2) {
                uint32_t rg[16], ru[16];
                tmem_ld16(tmem + lane_base + kColAcc + buf * 32, rg);
                tmem_ld16(tmem + lane_base + kColAcc + buf * 32 + 16, ru);
                tmem_ld_wait();
#pragma unroll
                for (int t = 0; t < kMaxRows; ++t) {
                    if (t < n_tok) {
                        const float a1 = m.s[t];
                        const float g = bf16_round(__uint_as_float(rg[t]) * a1), up = bf16_round(__uint_as_float(ru[t]) * a1);
                        zs[t * 129 + mrow] = ((g / (1.0f + expf(-g))) * up) * m.c;
                    }
                }
                bar_sync(1, 128);
                const int t = te >> 3, gi = te & 7;
                if (t < n_tok) {
                    float z[16];
                    float amax = 0.f;
#pragma unroll
                    for (int k = 0; k < 16; ++k) {
                        z[k] = zs[t * 129 + gi * 16 + k];
                        amax = fmaxf(amax, fabsf(z[k]));
                    }
                    const int eg = prov_exp_u(amax);
                    const float down = __uint_as_float((uint32_t)(127 - eg) << 23);
                    const uint32_t sfb = float_to_e4m3((amax * down) * (1.0f / 6.0f));
                    const float d = e4m3_to_float(sfb);
                    const float inv = d > 0.f ? 1.0f / d : 0.f;
                    uint32_t lo = 0, hi = 0;
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        lo |= float_to_e2m1((z[k] * down) * inv) << (4 * k);
                        hi |= float_to_e2m1((z[8 + k] * down) * inv) << (4 * k);
                    }
                    const int slot = m.slot[t], gcol = (a.rank * a.I_s + blk * 128) / 16 + gi;
                    for (int p = 0; p < a.n_peer; ++p) {
                        *(uint2*)(a.z_peer[p] + (size_t)slot * (a.I / 2) + gcol * 8) = make_uint2(lo, hi);
                        a.zsf_peer[p][(size_t)slot * (a.I / 16) + gcol] = (unsigned char)sfb;
                        a.zex_peer[p][(size_t)slot * (a.I / 16) + gcol] = (signed char)eg;
                    }
                }
                bar_sync(1, 128);
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
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2) tmem_dealloc(tmem, kTmemCols);
}

size_t experts_umma_smem(bool g2) {
    const size_t stage = (g2 ? 1 : 2) * (size_t)(kTileBytes + kSfBytes);
    const int S = g2 ? 10 : 5;
    return 1024 + S * stage + kMaxKChunks * 2048 + (16 * 129 + 1) * 4 + 2 * sizeof(UnitMeta) + 16 + (2 * S + 5) * 8 + 16;
}

cudaError_t experts_umma_prepare() {
    cudaError_t e = cudaFuncSetAttribute(experts_umma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)experts_umma_smem(false));
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(experts_umma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)experts_umma_smem(true));
}

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
