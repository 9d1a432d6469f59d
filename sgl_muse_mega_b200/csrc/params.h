// Types shared by the layer's kernels and the host launcher: limits, route tables, the GEMM argument record.
#pragma once

#include <stdint.h>

#include "util.cuh"

namespace mk {

constexpr int kMaxRanks = 8;
constexpr int kMaxRows = 16;
constexpr int kMaxSlots = 128;  // rows x topk
constexpr int kHeadDim = 64;

// Route tables in the private scratch, written by the front kernel each launch.
struct RouteTables {
    int n_active;                   // distinct routed experts
    int act_e[kMaxSlots];           // their ids, ascending
    int act_off[kMaxSlots + 1];     // first sorted slot of each (exclusive scan of the counts)
    int slot[kMaxSlots];            // sorted position -> slot index (token x topk + k)
};

struct GemmArgs {
    const void* w;        // [N, K] row-major weights (bf16 or f32)
    const void* x;        // [M, K] row-major activations (bf16, or f32 for f32 weights)
    int M, N, K;
    int ldw, ldx;         // row strides in elements
    float* partial;       // [ksplit, 16, N] f32 partial sums (ksplit > 1)
    unsigned* counter;    // [N / BN] arrival counters (zero between launches)
    void* out[kMaxRanks]; // destinations (own buffer and peers'), each [M, ldo]
    int n_out;
    int ldo;              // row stride of out in elements
    int col0;             // first output column of this N range
    int out_f32;          // 1: f32 outputs, 0: bf16
};


}  // namespace mk
