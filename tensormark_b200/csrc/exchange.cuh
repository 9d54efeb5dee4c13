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

// Bounded wait until a flag that a peer GPU raises has reached `want`.
__device__ __forceinline__ bool wait_flag(const int* flag, int want) {
    auto peek = [&]() { int v; asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory"); return v; };
    if (peek() - want >= 0) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 32; ++i)
            if (peek() - want >= 0) return true;
        if (global_ns() - t0 > kWaitLimitNs) return false;
    }
}
// Consumer side of the exchange: one thread waits for every other rank's flag, the CTA follows.
__device__ __forceinline__ void exchange_wait(const Exchange& xc, int* status) {
    if (!xc.nwait) return;
    if (threadIdx.x == 0) {
        const int want = *(volatile const int*)xc.epoch + 1;
        bool ok = true;
        for (uint32_t q = 0; q < xc.nwait; ++q)
            if (q != xc.self) ok = wait_flag(xc.wait_flags + q, want) && ok;
        if (!ok) *(volatile int*)status = 2;
    }
    __syncthreads();
}

}  // namespace tmc
