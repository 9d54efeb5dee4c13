// common.cuh — shared declarations of the CUDA translation units.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

namespace tmc {

// dtype ids of the weight container (tensormark/tmq.h:48-60)
enum : unsigned { DT_Q8_0 = 0, DT_Q4_0 = 1, DT_F16 = 3, DT_Q4_1 = 4, DT_Q5_K = 5, DT_Q6_K = 6 };

inline __host__ __device__ unsigned block_elems(unsigned dt) {
    return (dt == 0 || dt == 1 || dt == 4) ? 32u : (dt == 5 || dt == 6) ? 256u : 0u;
}
inline __host__ __device__ unsigned block_bytes(unsigned dt) {
    switch (dt) { case 0: return 34; case 1: return 18; case 4: return 20; case 5: return 176; case 6: return 210; default: return 0; }
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
int* device_status_word();                  // device int the kernels write a nonzero code to when a bounded wait ran out

constexpr int kMaxSeg = 16;
struct SegTable {                           // rows [row_end[s-1], row_end[s]) start at byte woff[s]
    uint64_t woff[kMaxSeg];
    uint32_t row_end[kMaxSeg];
    uint32_t nseg;
};

// ---- kernel launchers (one per .cu) -----------------------------------------
struct GemvFuse {                           // optional fusions of the decode chain
    unsigned x_op;                          // 0 none, 1 rmsnorm (x2 = weights, eps), 2 silu(x) * x2
    const float* x2;
    float eps;
    bool accumulate;                        // y[row] += dot instead of y[row] = dot
};
bool launch_gemv(const float* x, const uint8_t* W, float* y, unsigned N, unsigned K, unsigned dtype,
                 const SegTable& seg, cudaStream_t st, const GemvFuse* fuse = nullptr);
bool launch_dequant(const uint8_t* W, float* out, unsigned N, unsigned K, unsigned dtype, cudaStream_t st);
bool launch_dequant_half(const uint8_t* W, void* out_half, unsigned N, unsigned K, unsigned dtype, cudaStream_t st);

}  // namespace tmc
