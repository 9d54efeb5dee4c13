// tests/host/host_contracts.cpp — exercises the host-side headers under include/.
//
// Built as a small shared library by the CPU test-suite (g++ -std=c++23
// -ffp-contract=off). It checks the three host contracts a caller of the reference
// compiles against: the block structs and scalar dequantizers (quant.h), the
// per-tensor projection strategy (q4_projection_backend.h; the assertions follow
// the reference's own test_q4_projection_backend.cpp:22-38) and the row-chunk pool
// (gemv_pool.h).
#include "quant.h"
#include "q4_projection_backend.h"
#include "gemv_pool.h"

#include <cstring>
#include <vector>

namespace {
int gemv_calls = 0, gemm_calls = 0;
bool fake_gemv(const float* x, const void* w, float* y, unsigned rows, unsigned cols) {
    ++gemv_calls;
    if (!(x && w && y && rows == 4 && cols == 32)) return false;
    y[0] = 7.f;
    return true;
}
bool fake_gemm(const float* x, const void* w, float* y, unsigned batch, unsigned rows, unsigned cols) {
    ++gemm_calls;
    if (x && w && y && batch == 8 && rows == 4 && cols == 32) y[0] = 9.f;
    return false;                       // a refused dispatch must reach the caller as false
}

struct PoolCtx { std::uint32_t dtype; };
thread_local std::vector<float> row_buf;
std::uint32_t g_dtype = 0;
void pool_kernel(const tmllama::GemvArgs& a, int o0, int o1) {
    const std::size_t rb = tmq::weight_bytes(g_dtype, 1, (std::size_t)a.n_in);
    if (row_buf.size() < (std::size_t)a.n_in) row_buf.resize((std::size_t)a.n_in);
    for (int o = o0; o < o1; ++o) {
        tmq::dequantize_row(g_dtype, static_cast<const std::uint8_t*>(a.w) + (std::size_t)o * rb, row_buf.data(), (std::size_t)a.n_in);
        float acc = 0.f;
        for (int k = 0; k < a.n_in; ++k) acc += row_buf[(std::size_t)k] * a.x[(std::size_t)k];
        a.y[(std::size_t)o] = acc;      // global row index into the BASE pointer
    }
}
}  // namespace

#include "tmq_reader.h"

extern "C" {
// .tmq container: number of tensors of a file, or -1 when the reader rejects it
__attribute__((visibility("default"))) int hc_tmq_count(const char* path) {
    tmmq::Mapped m;
    if (!m.open(path)) return -1;
    return (int)m.tensors().size();
}
// one tensor by name: dtype, nblocks, payload offset in the file, rank and up to 4 dims; 0 when absent
__attribute__((visibility("default"))) int hc_tmq_tensor(const char* path, const char* name, unsigned* dtype, unsigned long long* nblocks,
                                                         unsigned long long* payload, unsigned* rank, unsigned* dims) {
    tmmq::Mapped m;
    if (!m.open(path)) return 0;
    const tmmq::TensorInfo* t = m.find(name);
    if (!t) return 0;
    *dtype = t->dtype; *nblocks = t->nblocks; *payload = (unsigned long long)(t->blocks - m.base()); *rank = (unsigned)t->shape.size();
    for (std::size_t i = 0; i < t->shape.size() && i < 4; ++i) dims[i] = t->shape[i];
    return 1;
}
__attribute__((visibility("default"))) int hc_dequant(unsigned dtype, const void* blocks, float* out, std::size_t n) {
    try { tmq::dequantize_row(dtype, blocks, out, n); return 1; } catch (...) { return 0; }
}
__attribute__((visibility("default"))) float hc_fp16_to_fp32(std::uint16_t h) { return tmq::fp16_to_fp32(h); }
__attribute__((visibility("default"))) std::uint16_t hc_fp32_to_fp16(float f) { return tmq::fp32_to_fp16(f); }
__attribute__((visibility("default"))) std::size_t hc_weight_bytes(unsigned dtype, std::size_t out, std::size_t in) { return tmq::weight_bytes(dtype, out, in); }

// 0 when every assertion of the strategy contract holds, else the number of the first that failed.
__attribute__((visibility("default"))) int hc_strategy_selftest() {
    using namespace tmllama;
    gemv_calls = gemm_calls = 0;
    float input[32] = {}, output[4] = {};
    int weights = 0;
    const Q4ProjectionOps gpu{fake_gemv, fake_gemm};
    const auto cpu = make_q4_projection_strategy(false, gpu);
    if (cpu.supports(1) || cpu.run(input, &weights, output, 1, 4, 32)) return 1;
    if (gemv_calls != 0 || gemm_calls != 0) return 2;
    const auto sel = make_q4_projection_strategy(true, gpu);
    if (!sel.supports(1) || !sel.supports(8)) return 3;
    if (!sel.run(input, &weights, output, 1, 4, 32)) return 4;
    if (output[0] != 7.f || gemv_calls != 1 || gemm_calls != 0) return 5;
    if (sel.run(input, &weights, output, 8, 4, 32)) return 6;
    if (output[0] != 9.f || gemm_calls != 1) return 7;
    if (sel.supports(0) || sel.run(input, &weights, output, 0, 4, 32)) return 8;
    if (sel.supports(-3)) return 9;
    if (make_q4_projection_strategy(true, {fake_gemv, nullptr}).supports(8)) return 10;
    if (make_q4_projection_strategy(true, {nullptr, fake_gemm}).supports(1)) return 11;
    return 0;
}

__attribute__((visibility("default"))) int hc_pool_gemv(unsigned dtype, const void* W, const float* x, float* y, int n_out, int n_in, int threads) {
    try {
        tmllama::GemvPool pool(threads);
        g_dtype = dtype;
        tmllama::GemvJob j;
        j.kern = pool_kernel;
        j.a.w = W;
        j.a.x = std::span<const float>(x, (std::size_t)n_in);
        j.a.y = std::span<float>(y, (std::size_t)n_out);
        j.a.n_in = n_in;
        j.n_out = n_out;
        pool.dispatch(j);
        pool.dispatch(j);               // a pool is reusable
        tmllama::GemvJob bad = j;
        bad.kern = nullptr;
        try { pool.dispatch(bad); return -1; } catch (const std::invalid_argument&) {}
        return pool.nthreads;
    } catch (...) { return -2; }
}
}
