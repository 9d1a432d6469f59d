// Types shared by the layer's kernels and the host launcher: limits, route tables, the GEMM argument record.
#pragma once

#include <stdint.h>

#include "util.cuh"

namespace mk {

constexpr int kMaxRanks = 8;
constexpr int kMaxRows = 16;
constexpr int kMaxSlots = 128;  // rows x topk
constexpr int kHeadDim = 64;

// Route tables in the private scratch, written by the routing kernel each launch.
struct RouteTables {
    int n_active;                   // distinct routed experts
    int act_e[kMaxSlots];           // their ids, ascending
    int act_off[kMaxSlots + 1];     // first sorted slot of each (exclusive scan of the counts)
    int slot[kMaxSlots];            // sorted position -> slot index (token x topk + k)
};

// One skinny GEMM out[m, n] = sum_k x[m, k] W[n, k] (gemm.cu). `mode` 1 adds the qkv row ops to the epilogue.
struct GemmArgs {
    const void* w;        // [N, K] row-major weights (bf16 or f32)
    const void* x;        // [M, K] row-major activations (bf16, or f32 for f32 weights)
    int M, N, K;
    int ldw, ldx;         // row strides in elements
    int wn;               // 16-row groups per CTA: 1, 2 or 4 (the tile is 16 wn rows)
    int ksplit;           // K slices = cluster size along grid y (1, 2, 4, 8)
    void* out[kMaxRanks]; // destinations (own buffer and peers'), each [M, ldo]
    int n_out;
    int ldo;              // row stride of out in elements
    int col0;             // first output column of this N range
    int out_f32;          // 1: f32 outputs, 0: bf16
    // mode 1: the tile is one 64-wide head of a [q | k | v | o-gate] row: qk norm, q scale, RoPE, K/V append
    int mode;
    const float* cos_sin;
    const int* cache_loc;
    unsigned char* k_cache;
    unsigned char* v_cache;
    float q_scale, eps;
    int qh, kvh, kv_row_bytes;
    int* status;          // the launch's status block (a bulk copy that never lands records itself); may be null
};

}  // namespace mk
