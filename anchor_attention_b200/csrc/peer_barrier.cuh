// Barrier between the ranks of a head-parallel layer, after step 3 has stored its output
// rows into every rank's copy: each rank announces "epoch e reached" in every peer's flag
// array and then waits until every peer has announced it in its own.  Plain peer stores and
// loads with release / acquire semantics at system scope; nothing is multicast, nothing is
// reduced in the switch.  (The reference is single-GPU, test_hf.py:126: no counterpart.)
//
// The wait is bounded by time: a peer that never arrives (a rank that left or failed
// between steps) makes the kernel give up after `timeout_ns`, set the status word and
// return, so the surviving ranks' GPUs stay usable and their hosts can read the error.
#pragma once
#include <stdint.h>

namespace aa {

constexpr int kBarrierMaxPeers = 8;

struct PeerBarrierArgs {
    int32_t* flags[kBarrierMaxPeers];   // flags[p]: rank p's array of n_peers int32 (peer-mapped for p != rank)
    int n_peers, rank;
    int32_t epoch;                      // strictly increasing from call to call, the same on every rank
    unsigned long long timeout_ns;
    int32_t* status;                    // set to 1 when a wait gave up
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// one block of kBarrierMaxPeers threads; thread p talks to peer p
__global__ void __launch_bounds__(32) peer_barrier_kernel(PeerBarrierArgs a) {
    const int p = threadIdx.x;
    if (p >= a.n_peers) return;
    // everything this GPU stored before (the output rows of step 3) is ordered before the flag
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(a.flags[p] + a.rank), "r"(a.epoch) : "memory");
    const int32_t* mine = a.flags[a.rank] + p;
    const unsigned long long t0 = global_timer_ns();
    for (unsigned int i = 0;; ++i) {
        int32_t v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if ((int32_t)((uint32_t)v - (uint32_t)a.epoch) >= 0) return;     // epochs only grow (wrap-safe)
        if (i > 64) __nanosleep(200);
        if ((i & 63) == 63 && global_timer_ns() - t0 > a.timeout_ns) break;
    }
    atomicMax(a.status, 1);
}

}  // namespace aa
