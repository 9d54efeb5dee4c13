// exchange.cuh — device side of the peer-memory all-gather that row-sharded models fuse into their
// kernels (struct Exchange in common.cuh): bounded waits on flags that other GPUs raise.
#pragma once

#include "common.cuh"

namespace tmc {

constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // what has not happened within 2 s never will

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait until a counter that a peer GPU increments has reached `want` (wrap-safe comparison).
__device__ __forceinline__ bool wait_counter(const unsigned* ctr, unsigned want) {
    auto peek = [&]() { unsigned v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory"); return v; };
    if ((int)(peek() - want) >= 0) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 32; ++i)
            if ((int)(peek() - want) >= 0) return true;
        if (global_ns() - t0 > kWaitLimitNs) return false;
    }
}
// Consumer side of the exchange: one thread waits for every other rank's counter, the CTA follows.
__device__ __forceinline__ void exchange_wait(const Exchange& xc, int* status) {
    if (!xc.nwait) return;
    if (threadIdx.x == 0) {
        const unsigned want = (unsigned)(*(volatile const int*)xc.epoch + 1) * xc.wait_ctas;
        bool ok = true;
        for (uint32_t q = 0; q < xc.nwait; ++q)
            if (q != xc.self) ok = wait_counter(xc.wait_ctrs + q, want) && ok;
        if (!ok) *(volatile int*)status = 2;
    }
    __syncthreads();
}
// Producer side, end of a CTA: every row this CTA computed has been stored here and on the peers by the
// threads that computed it; after the barrier one thread adds this CTA to the rank's counter on every peer.
// A system-scope fence before the (relaxed) reductions orders the rows before every count: a peer that sees the
// count sees the rows. One fence for all peers, where a release per peer waited for the stores once per peer.
__device__ __forceinline__ void exchange_signal(const Exchange& xc) {
    if (!xc.npush) return;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();                                 // one wait for the rows on every peer, then the counts
        for (uint32_t q = 0; q < xc.npush; ++q)
            asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(xc.peer_ctr[q]) : "memory");
    }
}

}  // namespace tmc
