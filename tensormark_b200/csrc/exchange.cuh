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

__device__ __forceinline__ int peek_word(const int* p) {
    int v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Bounded wait until a counter that a peer GPU increments has reached `want` (wrap-safe comparison). Gives up
// when `limit_ns` has passed or when the abort word (may be null) is raised by whoever gave up first.
__device__ __forceinline__ bool wait_counter(const unsigned* ctr, unsigned want, unsigned long long limit_ns, const int* abort_word) {
    auto peek = [&]() { unsigned v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory"); return v; };
    if ((int)(peek() - want) >= 0) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 32; ++i)
            if ((int)(peek() - want) >= 0) return true;
        if (abort_word && peek_word(abort_word)) return false;
        if (global_ns() - t0 > limit_ns) return false;
    }
}
// Consumer side of the exchange: one thread waits for every other rank's counter, the CTA follows. The first
// wait that runs out writes status 2 and raises the abort word here and on every peer; while it is up no wait
// is attempted at all (the data read afterwards is incomplete, which the status word tells the host).
// The wait itself, for ONE thread; false when it gave up (status and abort words are then set).
__device__ __forceinline__ bool exchange_wait_thread(const Exchange& xc, int* status) {
    if (!xc.nwait) return true;
    bool ok = !(xc.abort_local && peek_word(xc.abort_local));
    if (ok) {
        const unsigned want = (unsigned)(*(volatile const int*)xc.epoch + 1) * xc.wait_ctas;
        for (uint32_t q = 0; q < xc.nwait && ok; ++q)
            if (q != xc.self) ok = wait_counter(xc.wait_ctrs + q, want, xc.limit_ns, xc.abort_local);
    }
    if (!ok) {
        *(volatile int*)status = 2;
        if (xc.abort_local) {
            *(volatile int*)xc.abort_local = 1;
            for (uint32_t q = 0; q < xc.npeers; ++q) *(volatile int*)xc.abort_peer[q] = 1;
            __threadfence_system();
        }
    }
    return ok;
}
__device__ __forceinline__ void exchange_wait(const Exchange& xc, int* status) {
    if (!xc.nwait) return;
    if (threadIdx.x == 0) (void)exchange_wait_thread(xc, status);
    __syncthreads();
}
// Producer side, end of a CTA: every row this CTA computed has been stored here and on the peers by the
// threads that computed it; after the barrier one thread adds this CTA to the rank's counter on every peer.
// The barrier makes every thread's row stores happen-before thread 0's fence, and the system-scope fence orders
// them (by cumulativity) before the relaxed reductions that follow: a peer that sees the count sees the rows.
// Removing the fence loses exactly that order. One fence for all peers, where a release per peer waited for the
// stores once per peer.
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
