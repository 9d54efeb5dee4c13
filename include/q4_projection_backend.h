// include/q4_projection_backend.h — per-tensor Q4 projection contract.
//
// Same names, signatures and semantics as the reference's strategy header
// (tensormark/q4_projection_backend.h:7-43): a backend supplies a GEMV for one
// activation row and a GEMM for a batch; the strategy routes by batch size and
// reports false when it has nothing to run, when the batch is empty or negative,
// or when the backend itself refused. tm_cuda_q4_gemv / tm_cuda_sgemm_q4
// (include/cuda_shim.h) are the CUDA callbacks; cuda_q4_projection_ops() wires
// them in exactly as the reference wires the Metal pair (llama.h:3972-3976).
#pragma once

#include "cuda_shim.h"

namespace tmllama {

using Q4Gemv = bool (*)(const float* x, const void* weights, float* y, unsigned rows, unsigned cols);
using Q4Gemm = bool (*)(const float* x, const void* weights, float* y, unsigned batch, unsigned rows,
                        unsigned cols);

struct Q4ProjectionOps {
    Q4Gemv gemv = nullptr;
    Q4Gemm gemm = nullptr;
};

class Q4ProjectionStrategy {
public:
    constexpr explicit Q4ProjectionStrategy(Q4ProjectionOps ops = {}) : ops_(ops) {}

    // batch 1 needs a GEMV, larger batches need a GEMM, anything else is unsupported
    [[nodiscard]] constexpr bool supports(int batch) const noexcept {
        if (batch < 1) return false;
        return batch == 1 ? ops_.gemv != nullptr : ops_.gemm != nullptr;
    }

    [[nodiscard]] bool run(const float* x, const void* weights, float* y, int batch, int rows, int cols) const {
        if (!supports(batch)) return false;
        const unsigned r = static_cast<unsigned>(rows), c = static_cast<unsigned>(cols);
        return batch == 1 ? ops_.gemv(x, weights, y, r, c)
                          : ops_.gemm(x, weights, y, static_cast<unsigned>(batch), r, c);
    }

private:
    Q4ProjectionOps ops_;
};

// A disabled GPU yields a strategy with no callbacks, which supports nothing.
[[nodiscard]] constexpr Q4ProjectionStrategy make_q4_projection_strategy(bool gpu_enabled,
                                                                         Q4ProjectionOps gpu_ops) noexcept {
    return gpu_enabled ? Q4ProjectionStrategy(gpu_ops) : Q4ProjectionStrategy();
}

// The CUDA backend's callbacks.
[[nodiscard]] inline Q4ProjectionOps cuda_q4_projection_ops() noexcept {
    return Q4ProjectionOps{&tm_cuda_q4_gemv, &tm_cuda_sgemm_q4};
}

}  // namespace tmllama
