// common.cuh — shared declarations of the CUDA translation units.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

namespace tmc {

// dtype ids of the weight container (tensormark/tmq.h:48-60)
enum : unsigned { DT_Q8_0 = 0, DT_Q4_0 = 1, DT_F16 = 3, DT_Q4_1 = 4, DT_Q5_K = 5, DT_Q6_K = 6, DT_Q4_K = 8 };

inline __host__ __device__ unsigned block_elems(unsigned dt) {
    return (dt == 0 || dt == 1 || dt == 4) ? 32u : (dt == 5 || dt == 6 || dt == 8) ? 256u : 0u;
}
inline __host__ __device__ unsigned block_bytes(unsigned dt) {
    switch (dt) { case 0: return 34; case 1: return 18; case 4: return 20; case 5: return 176; case 6: return 210; case 8: return 144; default: return 0; }
}
inline size_t weight_bytes(unsigned dt, size_t n_out, size_t n_in) {
    const unsigned e = block_elems(dt);
    return (e == 0 || n_in % e) ? 0 : n_out * (n_in / e) * (size_t)block_bytes(dt);
}

// Error and launch bookkeeping (defined in cuda_shim.cu).
bool fail(const char* fmt, ...);            // records the message, bumps the fallback counter, returns false
void note_launch(unsigned n = 1);           // counts kernels launched by this library
bool check_launch(const char* what);        // cudaGetLastError -> fail()
int device_sm_count();
int* device_status_word();
// Kernel timeline (off unless TM_CUDA_TRACE=1): CTA 0 of every GEMV stamps %globaltimer at its start, after
// the wait for its predecessor, after x is staged and at its end, plus its shape: kTraceWords words per launch.
constexpr int kTraceWords = 6, kTraceLaunches = 8192;
unsigned long long* device_trace();         // nullptr when tracing is off                  // device int the kernels write a nonzero code to when a bounded wait ran out

constexpr int kMaxSeg = 16;
struct SegTable {                           // rows [row_end[s-1], row_end[s]) start at byte woff[s]
    uint64_t woff[kMaxSeg];
    uint32_t row_end[kMaxSeg];
    uint32_t yoff[kMaxSeg];                 // element of y that receives the segment's first row (default: its first row index)
    uint32_t nseg;
};

// Peer-memory all-gather fused into the kernels of a row-sharded model (one process per GPU). A
// producer stores each finished row of y into the same place of every peer's copy of the buffer as
// well as its own; when a CTA is done it adds 1 to this rank's counter of the gather "site" in every
// peer's memory (a release at system scope, so the rows are visible before the count). A consumer
// waits until the site's counters of all other ranks have reached epoch * ctas, where ctas is the
// producer's grid size, before it reads the gathered vector. Counters only grow, every wait is bounded
// and reports through the status word.
constexpr int kMaxPeers = 7;
struct Exchange {
    const int* epoch;                       // device int; the current token's epoch is *epoch + 1
    const unsigned* wait_ctrs;              // consumer: the site's counters in local memory, one per rank
    uint32_t nwait, self;                   // consumer: ranks (0 = no wait) and this rank's index
    uint32_t wait_ctas;                     // consumer: CTAs of the producing launch (arrivals per epoch and rank)
    uint32_t npush;                         // producer: number of peers (0 = no push)
    float* peer_y[kMaxPeers];               // producer: y as mapped from each peer
    unsigned* peer_ctr[kMaxPeers];          // producer: this rank's counter of the site in each peer's memory
};
unsigned last_gemv_grid();                  // CTAs of the most recent GEMV launch of this process

// ---- kernel launchers (one per .cu) -----------------------------------------
struct GemvFuse {                           // optional fusions of the decode chain
    unsigned x_op;                          // 0 none, 1 rmsnorm (x2 = weights, eps), 2 silu(x) * x2
    const float* x2;
    float eps;
    bool accumulate;                        // y[row] += dot instead of y[row] = dot
    const Exchange* xchg;                   // nullptr: single GPU
};
bool launch_gemv(const float* x, const uint8_t* W, float* y, unsigned N, unsigned K, unsigned dtype,
                 const SegTable& seg, cudaStream_t st, const GemvFuse* fuse = nullptr);
bool launch_dequant(const uint8_t* W, float* out, unsigned N, unsigned K, unsigned dtype, cudaStream_t st);
bool launch_dequant_half(const uint8_t* W, void* out_half, unsigned N, unsigned K, unsigned dtype, cudaStream_t st);

}  // namespace tmc
