// Device helpers shared by the layer's kernels: number formats, reductions, mma.sync wrappers, PDL wait.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mk {

typedef __nv_bfloat16 bf16;

// Programmatic dependent launch. `griddep_wait` blocks until the predecessor grid has completed and its writes are
// visible, THEN lets the successor grid start launching: the successor's CTAs fill SMs as this grid's CTAs retire and run
// their prologues (barrier setup, tensor-memory allocation, weight prefetch) under this grid's tail. Because the trigger
// comes after the wait, a successor's prologue may read anything written two or more kernels back, but nothing of its
// immediate predecessor before its own wait. Both are no-ops without the launch attribute.
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// (Measured the other way round, trigger first: the successors' CTAs then sit on the SMs while this grid still runs, and
// the layer takes 224 us instead of 215.)
__device__ __forceinline__ void griddep_wait_only() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() {
    griddep_wait_only();
    griddep_launch();
}

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum / max; `red` holds 33 floats of shared memory; every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float s = lane < nw ? red[lane] : 0.f;
        s = warp_sum(s);
        if (lane == 0) red[32] = s;
    }
    __syncthreads();
    return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float s = lane < nw ? red[lane] : -INFINITY;
        s = warp_max(s);
        if (lane == 0) red[32] = s;
    }
    __syncthreads();
    return red[32];
}

// A group of threads that works on one row together: the whole block (bar 0: __syncthreads) or the `n` threads of a
// warp-specialised kernel's epilogue warps that share named barrier `bar` (tid counts from the group's first thread).
struct Grp {
    int tid, n, bar;
};
__device__ __forceinline__ Grp block_grp() { return Grp{(int)threadIdx.x, (int)blockDim.x, 0}; }
__device__ __forceinline__ void grp_sync(const Grp& g) {
    if (g.bar == 0) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(g.bar), "r"(g.n) : "memory");
}
// Group-wide sum / max; `red` holds 33 floats of shared memory; every thread of the group gets the result.
__device__ __forceinline__ float grp_sum(float v, float* red, const Grp& g) {
    const int lane = g.tid & 31, warp = g.tid >> 5, nw = (g.n + 31) >> 5;
    v = warp_sum(v);
    grp_sync(g);
    if (lane == 0) red[warp] = v;
    grp_sync(g);
    if (warp == 0) {
        float s = lane < nw ? red[lane] : 0.f;
        s = warp_sum(s);
        if (lane == 0) red[32] = s;
    }
    grp_sync(g);
    return red[32];
}
__device__ __forceinline__ float grp_max(float v, float* red, const Grp& g) {
    const int lane = g.tid & 31, warp = g.tid >> 5, nw = (g.n + 31) >> 5;
    v = warp_max(v);
    grp_sync(g);
    if (lane == 0) red[warp] = v;
    grp_sync(g);
    if (warp == 0) {
        float s = lane < nw ? red[lane] : -INFINITY;
        s = warp_max(s);
        if (lane == 0) red[32] = s;
    }
    grp_sync(g);
    return red[32];
}

// ---- e2m1 / e4m3 ----

// 4-bit e2m1 code -> float: bit 3 sign, {0,.5,1,1.5,2,3,4,6}
__device__ __forceinline__ float e2m1_to_float(uint32_t c) {
    const uint32_t ee = (c >> 1) & 3u, m = c & 1u;
    const float mag = ee == 0 ? 0.5f * (float)m : __uint_as_float(((ee + 126u) << 23) | (m << 22));
    return (c & 8u) ? -mag : mag;
}

// float -> e2m1 code, round to nearest, ties to the even code, saturate at 6 (cvt.rn.satfinite.e2m1x2.f32 semantics)
__device__ __forceinline__ uint32_t float_to_e2m1(float x) {
    const float a = fabsf(x);
    uint32_t c = (a > 0.25f) + (a >= 0.75f) + (a > 1.25f) + (a >= 1.75f) + (a > 2.5f) + (a >= 3.5f) + (a > 5.0f);
    return c | ((__float_as_uint(x) >> 28) & 8u);
}

__device__ __forceinline__ float e4m3_to_float(uint32_t b) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
    return __half2float(__half(h));
}
__device__ __forceinline__ uint32_t float_to_e4m3(float x) {
    return (uint32_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}

// An e4m3 scale byte times 2^-delta (delta >= 0): exponent-field move while the result stays normal, round half up on the
// subnormal grid (the h-row view of the experts' second GEMM: every group's scale is moved to the row's largest exponent;
// test/reference/muse_spark.py:447-491).
__device__ __forceinline__ uint32_t scale_down_byte(uint32_t byte, int delta) {
    const int ef = (int)(byte >> 3);
    if (ef > delta) return byte - ((uint32_t)delta << 3);
    const uint32_t sig = (byte & 7u) | (ef != 0 ? 8u : 0u);
    int sh = delta - ef + (ef != 0 ? 1 : 0);
    sh = min(max(sh, 0), 8);
    const uint32_t half = sh > 0 ? (1u << (sh - 1)) : 0u;
    return (sig + half) >> sh;
}

// ---- mma.sync ----

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_tf32_1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

// Philox4x32-10 (Salmon et al., SC'11): the sampled step's uniforms are the top 24 bits of word i % 4 of
// philox({iteration, stream, purpose, i / 4}, seed); purpose 0 the draft walk, 1 the accept.
__device__ __forceinline__ uint4 philox4x32(uint4 c, uint2 k) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const unsigned long long p0 = (unsigned long long)0xD2511F53u * c.x, p1 = (unsigned long long)0xCD9E8D57u * c.z;
        c = make_uint4((unsigned)(p1 >> 32) ^ c.y ^ k.x, (unsigned)p1, (unsigned)(p0 >> 32) ^ c.w ^ k.y, (unsigned)p0);
        k.x += 0x9E3779B9u;
        k.y += 0xBB67AE85u;
    }
    return c;
}
__device__ __forceinline__ float philox_uniform(unsigned long long seed, unsigned stream, unsigned iter, unsigned purpose, int i) {
    const uint4 r = philox4x32(make_uint4(iter, stream, purpose, (unsigned)i / 4), make_uint2((unsigned)seed, (unsigned)(seed >> 32)));
    const unsigned w = (i & 3) == 0 ? r.x : (i & 3) == 1 ? r.y : (i & 3) == 2 ? r.z : r.w;
    return (float)(w >> 8) * 0x1p-24f;
}

// Trace builds (-DROWS_TRACE): thread 0 of every CTA of a row or attention kernel stamps entry (0), programmatic wait
// returned (1) and end (2) into a per-translation-unit device array [kernel][CTA][4]; RT_READ defines the C function
// that copies it out.
#ifdef ROWS_TRACE
static __device__ unsigned long long g_rows_trace[8][160][4];
#define RT(kid, slot)                                                           \
    if (threadIdx.x == 0 && threadIdx.y == 0 && blockIdx.y == 0) {              \
        unsigned long long t_;                                                  \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                  \
        if (blockIdx.x < 160) g_rows_trace[(kid)][blockIdx.x][(slot)] = t_;     \
    }
#define RT_READ(name)                                                                                                   \
    extern "C" int name(void* dst) {                                                                                    \
        return cudaMemcpyFromSymbol(dst, mk::g_rows_trace, sizeof(unsigned long long) * 8 * 160 * 4) == cudaSuccess ? 0 : -1; \
    }
#else
#define RT(kid, slot)
#define RT_READ(name)
#endif

}  // namespace mk
