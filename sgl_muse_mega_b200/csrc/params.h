// Types shared by the layer's kernels and the host launcher: limits, route tables, the GEMM argument record.
#pragma once

#include <stdint.h>

#include "util.cuh"

namespace mk {

constexpr int kMaxRanks = 8;
constexpr int kMaxRows = 16;
constexpr int kMaxSlots = 128;  // rows x topk
constexpr int kHeadDim = 64;

// ---- cross-GPU exchange points -----------------------------------------------------------------------------------------
// A tensor-parallel world of one process per GPU synchronises each exchange (the kernels store their results straight
// into the peers' buffers) with one counter word per exchange point in every rank's flag block:
//   producer kernel   every CTA: stores, barrier, device-scope fence, arrive on a local counter; the last CTA advances the
//                     local epoch word, fences at system scope and adds 1 to the exchange's word on every rank that
//                     received data (own included);
//   consumer kernel   after its programmatic-launch wait, one thread per CTA polls its own word until it reaches
//                     epoch x contributors, at most `budget` polls; a wait that runs out records itself in the status
//                     block and the kernel carries on (its outputs are then meaningless, nothing hangs).
// The words only grow; a launch sequence replayed from a CUDA graph needs no host-side reset. All-zero records (the
// default) switch the mechanism off: a world emulated on one GPU orders its launches on the stream instead.
constexpr int kXchgPoints = 8;   // words [0, 8) of the flag block: exchange counters (written by peers)
constexpr int kXchgEpoch = 8;    // words [8, 16): this rank's epoch per exchange (local)
constexpr int kXchgDone = 16;    // words [16, 24): CTA arrival counters of the producers (local)
constexpr int kXchgTarget = 24;  // words [24, 32): the epoch a producer launch of this rank is about to complete (local)
constexpr int kXchgWords = 32;
// The fused kernels (fused.cuh) feed and consume an exchange inside one kernel, one arrival per finished tile: they count in
// words of their own, so that both protocols can serve launches on one flag block.
constexpr int kFusedFlag = 32;   // words [32, 40): arrivals per exchange point (written by peers)
constexpr int kFusedEpoch = 40;  // words [40, 48): completed launches that fed the exchange (local)

struct XchgSignal {
    unsigned* flag[kMaxRanks];  // the exchange's word on every receiving rank
    int n;                      // 0: off
    int remote;                 // some receiver is another rank (system-scope ordering needed)
    unsigned* done;
    unsigned* epoch;
    unsigned* target;           // xchg_announce: where the producer leaves epoch + 1 for a consumer that does not wait for its end
};
struct XchgWait {
    const unsigned* flag;       // this rank's word of the exchange; null: off
    const unsigned* epoch;
    unsigned contributors;      // signals per epoch
    long long budget;           // polls before giving up
    int* status;
    int stage;                  // recorded with a wait that ran out
    // packet mode (pkt_take_n below): the exchanged bf16 rows carry their own validity and there is no counter word
    int packets;                // 1: on (flag is null then)
    unsigned present;           // bit j: source j of the exchange is bound and writes its part (a part of an absent source is 0)
    int band;                   // columns per source where the sources write column bands of one row (0: whole rows)
    const unsigned* target;     // the epoch to wait for, left by this rank's producer launch (xchg_announce); null: the epoch word
};

// Every thread of every CTA calls this after the kernel's last store to a peer.
__device__ __forceinline__ void xchg_signal(const XchgSignal& x) {
    if (x.n == 0) return;
    __syncthreads();
    if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) {
        // Every CTA publishes its own stores at the scope of the receivers and arrives. With a peer among them that is a
        // system-scope fence per CTA: the CTAs pay it one by one as they finish, under the kernel's tail; the last CTA to
        // arrive has observed all of them and fences once more (nothing of its own is outstanding by then) before the
        // flag words. (A device-scope fence per CTA and one system-scope fence in the last CTA put the whole cost of
        // flushing the grid's peer stores behind the kernel's end.)
        if (x.remote) __threadfence_system();
        else __threadfence();
        const unsigned total = gridDim.x * gridDim.y * gridDim.z;
        if (atomicAdd(x.done, 1u) == total - 1) {
            *x.done = 0;
            *(volatile unsigned*)x.epoch = *(volatile unsigned*)x.epoch + 1;
            if (x.remote) {
                __threadfence_system();
                for (int i = 0; i < x.n; ++i) atomicAdd_system(x.flag[i], 1u);
            } else {  // the only receiver is this GPU: device scope is enough
                __threadfence();
                for (int i = 0; i < x.n; ++i) atomicAdd(x.flag[i], 1u);
            }
        }
    }
}

// A consumer kernel that does not wait for its own rank's producer grid to end cannot read the epoch word (the producer's
// last CTA advances it at some point while the consumer already runs). The producer's first CTA therefore leaves the epoch
// its launch will complete in the target word, after its own programmatic-launch wait (every earlier signal is in by
// then) and before it lets the dependent launch: thread 0 of CTA 0 calls this, the CTA synchronises, then triggers.
__device__ __forceinline__ void xchg_announce(const XchgSignal& x) {
    if (x.target == nullptr) return;
    *(volatile unsigned*)x.target = *(volatile unsigned*)x.epoch + 1;
    __threadfence();
}

// Every thread of every CTA calls this after griddep_wait() and before the first read of exchanged data.
// `epoch` is the exchange's epoch to wait for. A consumer kernel that runs after its own rank's producer kernel reads it
// from the epoch word (xchg_wait); a kernel that holds producer and consumer reads the word once at its start, before any
// of its CTAs can have signalled, and waits for that value + 1 (xchg_epoch / xchg_wait_epoch).
__device__ __forceinline__ unsigned xchg_epoch(const XchgWait& w) {
    return w.flag == nullptr ? 0u : *(volatile const unsigned*)w.epoch;
}
__device__ __forceinline__ void xchg_wait_epoch(const XchgWait& w, unsigned epoch) {
    if (w.flag == nullptr) return;
    if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) {
        const unsigned want = epoch * w.contributors;
        long long polls = 0;
#ifdef XCHG_TRACE
        unsigned long long t0_;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0_));
#endif
        for (;;) {
            unsigned seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(w.flag) : "memory");
            if ((int)(seen - want) >= 0) break;
            // a failure already on record (an earlier wait that ran out): do not wait a full budget again
            if ((polls & 1023) == 1023 && w.status != nullptr && *(volatile int*)w.status != 0) break;
            if (++polls > w.budget) {  // give up: record once per launch, never trap
                if (w.status != nullptr && atomicCAS(w.status, 0, 1) == 0) {
                    w.status[1] = w.stage;
                    w.status[2] = (int)blockIdx.x;
                    w.status[3] = (int)seen;
                    w.status[4] = (int)want;
                }
                break;
            }
            if (polls > 4096) __nanosleep(64);
        }
#ifdef XCHG_TRACE
        // trace builds: nanoseconds CTA 0 spent in this wait and the number of waits, per recorded stage (words 256.. of
        // the status block, as u64 pairs indexed by stage % 32)
        if (blockIdx.x == 0 && w.status != nullptr) {
            unsigned long long t1_;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1_));
            unsigned long long* acc_ = (unsigned long long*)(w.status + 256) + 2 * (w.stage & 31);
            acc_[0] += t1_ - t0_;
            acc_[1] += 1;
        }
#endif
    }
    __syncthreads();
}
__device__ __forceinline__ void xchg_wait(const XchgWait& w) { xchg_wait_epoch(w, xchg_epoch(w)); }

// The same wait for one role of a warp-specialised kernel: the `n` threads that share named barrier `bar` (tid counts from
// the role's first thread); the other roles carry on.
__device__ __forceinline__ void xchg_wait_role(const XchgWait& w, int tid, int n, int bar) {
    if (w.flag == nullptr) return;
    if (tid == 0) {
        const unsigned want = (w.target != nullptr ? *(volatile const unsigned*)w.target : xchg_epoch(w)) * w.contributors;
        long long polls = 0;
        for (;;) {
            unsigned seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(w.flag) : "memory");
            if ((int)(seen - want) >= 0) break;
            if ((polls & 1023) == 1023 && w.status != nullptr && *(volatile int*)w.status != 0) break;
            if (++polls > w.budget) {
                if (w.status != nullptr && atomicCAS(w.status, 0, 1) == 0) {
                    w.status[1] = w.stage;
                    w.status[2] = (int)blockIdx.x;
                    w.status[3] = (int)seen;
                    w.status[4] = (int)want;
                }
                break;
            }
            if (polls > 4096) __nanosleep(64);
        }
    }
    asm volatile("bar.sync %0, %1;" ::"r"(bar), "r"(n) : "memory");
}

// ---- packet mode: bf16 exchanges that carry their own validity --------------------------------------------------------------
// A bf16 whose 16 bits are all ones is a NaN that no float -> bf16 conversion produces (they give the canonical 0x7FFF), so an
// exchange buffer filled with it says, 2 bytes at a time, what has not arrived yet. The producers store their results into
// the peers' buffers as they finish a tile and do nothing else: no fence, no arrival count, no flag. A consumer thread polls
// the 16-byte packet it is about to use until none of its eight halves is the mark (stores of any width >= 2 bytes may
// complete it piecewise), takes the value and puts the mark back for the buffer's next use; that store is ordered before the
// next use because the peers reach it only through a later exchange that needs this rank's later kernels, which start after
// this one has ended. A poll that runs out of its budget records itself like a counter wait (code 1) and the kernel
// carries on with the bytes it saw.
constexpr unsigned kPktMark = 0xFFFFFFFFu;
__device__ __forceinline__ bool pkt_word_ok(unsigned w) { return (w & 0xFFFFu) != 0xFFFFu && (w >> 16) != 0xFFFFu; }
__device__ __forceinline__ bool pkt_ok(const uint4& v) {
    return pkt_word_ok(v.x) && pkt_word_ok(v.y) && pkt_word_ok(v.z) && pkt_word_ok(v.w);
}
__device__ __forceinline__ uint4 pkt_peek(const void* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
// One more poll of a thread: false when it has to give up (its budget ran out: recorded once per launch; or a failure is
// already on record, so that a launch gives up once and not once per wait).
__device__ __forceinline__ bool pkt_again(const XchgWait& w, long long& polls) {
    if ((polls & 255) == 255 && w.status != nullptr && *(volatile int*)w.status != 0) return false;
    if (++polls > w.budget) {
        if (w.status != nullptr && atomicCAS(w.status, 0, 1) == 0) {
            w.status[1] = w.stage;
            w.status[2] = (int)blockIdx.x;
            w.status[3] = (int)threadIdx.x;
            w.status[4] = -1;
        }
        return false;
    }
    return true;  // no sleep between rounds: a 32 ns sleep cost 1.3 us at the post norm, where the last rows decide
}
// The thread's n <= N packets at addr(0) .. addr(n - 1), those whose bit in `need` is set (the others read as zeros): all
// loads of a round are issued together (one memory round trip a round, not one a packet), the round repeats until every
// packet is whole; then the marks go back.
template <int N, class Addr>
__device__ __forceinline__ void pkt_take_n(uint4 (&v)[N], int n, unsigned need, Addr addr, const XchgWait& w) {
    long long polls = 0;
    for (;;) {
        bool ok = true;
#pragma unroll
        for (int j = 0; j < N; ++j)
            if (j < n && ((need >> j) & 1u)) {
                v[j] = pkt_peek(addr(j));
                ok = ok && pkt_ok(v[j]);
            }
        if (ok || !pkt_again(w, polls)) break;
    }
#pragma unroll
    for (int j = 0; j < N; ++j)
        if (j < n) {
            if ((need >> j) & 1u) *(uint4*)addr(j) = make_uint4(kPktMark, kPktMark, kPktMark, kPktMark);
            else v[j] = make_uint4(0, 0, 0, 0);
        }
}
// whether the source that writes column c of a row is present (bands of w.band columns a source; 0: whole rows, always)
__device__ __forceinline__ bool pkt_col_present(const XchgWait& w, int c) {
    return w.band <= 0 || ((w.present >> (c / w.band)) & 1u);
}

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
    XchgSignal sig;       // the exchange this GEMM's peer stores feed (off when n == 0)
    // the router only: score[m, n] = f32(sigmoid_f64(out[m, n] x score_mult)) + score_bias[n], the routing's selection scores
    float* score;
    const float* score_bias;
    double score_mult;
};

}  // namespace mk
