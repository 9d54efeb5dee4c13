// common.cuh — shared declarations of the CUDA translation units.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

namespace tmc {

// dtype ids of the weight container (tensormark/tmq.h:48-60)
// 9 is GGUF's own Q4_0 block: the same 18 bytes with SPLIT nibbles (byte j = elements j | j + 16, llama.h:4588-4597),
// where the container's Q4_0 interleaves (byte j = elements 2j | 2j + 1). 3 and 10 are plain fp16 / bf16 rows, served by
// gemv_f16.cu; they are not block formats (block_elems is 0 for them).
// 7 is the ternary pack TQ2: 128 two-bit codes and one fp16 scale per 34-byte block, w = (code - 1) * d (quant.h:446-566).
enum : unsigned { DT_Q8_0 = 0, DT_Q4_0 = 1, DT_F16 = 3, DT_Q4_1 = 4, DT_Q5_K = 5, DT_Q6_K = 6, DT_TQ2 = 7, DT_Q4_K = 8, DT_GGUF_Q4_0 = 9, DT_BF16 = 10 };

inline __host__ __device__ unsigned block_elems(unsigned dt) {
    return (dt == 0 || dt == 1 || dt == 4 || dt == 9) ? 32u : (dt == 5 || dt == 6 || dt == 8) ? 256u : dt == 7 ? 128u : 0u;
}
inline __host__ __device__ unsigned block_bytes(unsigned dt) {
    switch (dt) { case 0: case 7: return 34; case 1: case 9: return 18; case 4: return 20; case 5: return 176; case 6: return 210; case 8: return 144; default: return 0; }
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
// well as its own; when a CTA is done (a barrier, then ONE system-scope fence, which orders the whole
// CTA's row stores before what follows) it adds 1 to this rank's counter of the gather "site" in every
// peer's memory with relaxed reductions. A consumer waits until the site's counters of all other ranks
// have reached epoch * ctas, where ctas is the producer's grid size, before it reads the gathered
// vector. Counters only grow and every wait is bounded (limit_ns). A wait that runs out sets the status
// word and a sticky abort word in this rank's arena and in every peer's: every later wait, here and
// there, returns at once instead of spending its own limit, so a stalled rank costs one limit, not one
// per kernel. The host clears the abort word when it harvests the status.
constexpr int kMaxPeers = 7;
struct Exchange {
    const int* epoch;                       // device int; the current token's epoch is *epoch + 1
    const unsigned* wait_ctrs;              // consumer: the site's counters in local memory, one per rank
    uint32_t nwait, self;                   // consumer: ranks (0 = no wait) and this rank's index
    uint32_t wait_ctas;                     // consumer: CTAs of the producing launch (arrivals per epoch and rank)
    uint32_t npush;                         // producer: number of peers (0 = no push)
    float* peer_y[kMaxPeers];               // producer: y as mapped from each peer
    unsigned* peer_ctr[kMaxPeers];          // producer: this rank's counter of the site in each peer's memory
    unsigned long long limit_ns;            // consumer: how long one wait may last
    int* abort_local;                       // sticky abort word of this rank's arena (nullptr: none)
    int* abort_peer[kMaxPeers];             // the same word in each peer's arena
    uint32_t npeers;
};
unsigned last_gemv_grid();                  // CTAs of the most recent GEMV launch of this process

// x in the GEMV lanes' unit form, in global memory, written once per launch (xprep kernel) instead of once per CTA:
// kXqHeaderWords words of header ([0] = the RMSNorm factor as a float, 1.0 without a norm), then the units of
// Lane<dtype>. It pays where staging is heavy (SiLU*up over a long K); for K = 4096 the extra dependent kernel costs
// what it saves, and a variant in which the producing GEMV's last CTA staged its own output was slower still (two
// more dependent L2 round trips at the end of the producer): measured on the 8B decode chain, 2.24 / 2.03 / 1.94 ms
// per token with tails + staging kernels / staging kernels everywhere / neither.
constexpr int kXqHeaderWords = 16;
size_t xq_bytes(unsigned K, unsigned dtype);            // size of such an image; 0 for an unknown format

// ---- kernel launchers (one per .cu) -----------------------------------------
struct GemvFuse {                           // optional fusions of the decode chain
    unsigned x_op;                          // 0 none, 1 rmsnorm (x2 = weights, eps), 2 silu(x) * x2
    const float* x2;
    float eps;
    bool accumulate;                        // y[row] += dot instead of y[row] = dot
    const Exchange* xchg;                   // nullptr: single GPU
    const uint32_t* xq;                     // x (after x_op) already in unit form for this dtype and K; the fp32 x is
                                            // still passed: rows that are not 16-byte aligned take the plain kernel
};
// x (after x_op) in unit form for a GEMV of `dtype`; xchg: wait for a peer gather first.
bool launch_xprep(uint32_t* out, const float* x, const float* x2, unsigned x_op, float eps, unsigned K, unsigned dtype,
                  const Exchange* xchg, cudaStream_t st);
bool launch_gemv(const float* x, const uint8_t* W, float* y, unsigned N, unsigned K, unsigned dtype,
                 const SegTable& seg, cudaStream_t st, const GemvFuse* fuse = nullptr);
// gemv_f16.cu: plain 16-bit rows (fp16 or bf16), and the GGUF -> container Q4_0 nibble reorder
bool launch_gemv_half(const float* x, const void* W, float* y, unsigned N, unsigned K, bool bf16, cudaStream_t st);
bool launch_embed_half(const unsigned* tok, unsigned idx, const void* W, float* x, unsigned D, bool bf16, cudaStream_t st);
bool launch_q4_split_to_interleaved(uint8_t* blocks, size_t nblocks, cudaStream_t st);
bool launch_dequant(const uint8_t* W, float* out, unsigned N, unsigned K, unsigned dtype, cudaStream_t st);
bool launch_dequant_half(const uint8_t* W, void* out_half, unsigned N, unsigned K, unsigned dtype, cudaStream_t st);

}  // namespace tmc
