// gemm.h — launcher of the tensor-core prefill GEMM (gemm.cu).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace tmc {

// Device scratch the GEMM needs for an M-token batch against an N x K tensor.
size_t gemm_workspace_bytes(unsigned M, unsigned N, unsigned K);
// C[m * ldc + n] = sum_k A[m][k] * W[n][k]  for m < M, n < N; ldc >= N.
bool launch_gemm(const float* A, const uint8_t* W, float* C, unsigned ldc, unsigned M, unsigned N, unsigned K,
                 unsigned dtype, void* workspace, size_t workspace_bytes, cudaStream_t st);

// For callers that keep an fp16 copy of static weights: the copy (exact fp32 value of every weight rounded once, as the
// GEMM's own pre-pass writes it), and the GEMM against it, whose workspace only holds the rounded activations.
bool launch_weights_f16(const uint8_t* W, void* Wh, unsigned N, unsigned K, unsigned dtype, cudaStream_t st);
bool launch_gemm_hh(const void* Ah, const void* Wh, float* C, unsigned ldc, unsigned M, unsigned N, unsigned K, bool accumulate, cudaStream_t st);
// The gated FFN's first half in one launch: act[M][F] (fp16) = silu(A Wg^T) * (A Wu^T), Wgu [2 F][K] fp16 with gate row f
// at row 2f and up row f at row 2f + 1; the gate and up values stay in the kernel's epilogue.
bool launch_gemm_hh_silu_mul(const void* Ah, const void* Wgu, void* act, unsigned M, unsigned F, unsigned K, cudaStream_t st);
size_t gemm_f16w_workspace_bytes(unsigned M, unsigned K);
bool launch_gemm_f16w(const float* A, const void* Wh, float* C, unsigned ldc, unsigned M, unsigned N, unsigned K,
                      void* workspace, size_t workspace_bytes, cudaStream_t st);

}  // namespace tmc
