// cuda_shim.cu — library state and the per-tensor entry points of the C ABI.
//
// The CUDA counterpart of the reference's Metal shim (tensormark/metal_shim.mm:6-20)
// and of the device singleton behind it (tensormark/metal.h:73-91): one device, one
// stream, a sticky error string, a fallback counter (metal.h:46-59), and the
// pointer-keyed weight cache of the per-call entries (metal.h:1986-1998,
// 2064-2079, 2141-2164). The token lane lives in token_lane.cu.
#include "cuda_shim.h"
#include "common.cuh"
#include "state.h"
#include "gemm.h"

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace tmc {

State& state() {
    static State s;
    return s;
}

bool fail(const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    State& s = state();
    s.last_error = buf;
    ++s.fallbacks;
    if (s.verbose) std::fprintf(stderr, "[tm_cuda] %s\n", buf);
    return false;
}

void note_launch(unsigned n) { state().launches += n; }

bool check_launch(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return true;
    return fail("%s: %s", what, cudaGetErrorString(e));
}

int device_sm_count() { return state().sm_count; }
int* device_status_word() { return state().status_dev; }
unsigned long long* device_trace() { return state().trace_dev; }

bool ensure_init(int device) {
    State& s = state();
    if (s.ready) {
        if (device >= 0 && device != s.device) return fail("already initialised on device %d", s.device);
        return true;
    }
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail("no CUDA device: this library has no CPU path");
    }
    if (device < 0) {
        // Under a one-process-per-GPU launcher the local rank picks the device.
        const char* lr = std::getenv("LOCAL_RANK");
        device = lr ? std::atoi(lr) % count : 0;
    }
    if (device >= count) return fail("device %d out of range (%d present)", device, count);
    if (cudaSetDevice(device) != cudaSuccess) return check_launch("cudaSetDevice");
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return check_launch("cudaGetDeviceProperties");
    if (prop.major != 10) return fail("device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
    s.device = device;
    s.sm_count = prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) != cudaSuccess) return check_launch("cudaStreamCreate");
    // The status word lives in pinned host memory that the device sees: reading it after a synchronisation costs
    // nothing, where a 4-byte copy back cost about 10 us on every blocking call.
    void* hp = nullptr;
    if (cudaHostAlloc(&hp, 64, cudaHostAllocMapped) != cudaSuccess) return check_launch("cudaHostAlloc(status)");
    std::memset(hp, 0, 64);
    s.status_host = (volatile int*)hp;
    if (cudaHostGetDevicePointer((void**)&s.status_dev, hp, 0) != cudaSuccess) return check_launch("cudaHostGetDevicePointer(status)");
    const char* tr = std::getenv("TM_CUDA_TRACE");
    if (tr && *tr == '1') {
        const size_t words = 1 + (size_t)kTraceWords * kTraceLaunches;
        if (cudaMalloc(&s.trace_dev, words * 8) != cudaSuccess) return check_launch("cudaMalloc(trace)");
        cudaMemset(s.trace_dev, 0, words * 8);
    }
    const char* v = std::getenv("TM_CUDA_VERBOSE");
    s.verbose = v && *v == '1';
    const char* wl = std::getenv("TM_CUDA_WAIT_LIMIT_MS");
    if (wl && *wl && std::atoll(wl) > 0) s.wait_limit_ns = (unsigned long long)std::atoll(wl) * 1000000ull;
    const char* kh = std::getenv("TM_CUDA_KV_HALF");
    s.kv_half = !(kh && *kh == '0');
    s.ready = true;
    return true;
}

// Reads and clears the device status word the kernels set when a bounded wait ran out.
bool harvest_status(const char* where) {
    State& s = state();
    const int h = *s.status_host;                        // the caller has just synchronised with the kernels
    if (h != 0) {
        *s.status_host = 0;
        // lower this rank's sticky abort word, so that the next token's waits are real waits again
        if (s.peer.arena) cudaMemsetAsync((int*)s.peer.arena + kAbortWord, 0, sizeof(int), s.stream);
        return fail("%s: a kernel gave up on a bounded wait (status %d)", where, h);
    }
    return true;
}

bool sync_stream(cudaStream_t st, const char* where) {
    const cudaError_t e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail("%s: %s", where, cudaGetErrorString(e));
    return harvest_status(where);
}

// ---- scratch: grow-only device buffers owned by the library -------------------
void* Scratch::get(size_t bytes) {
    if (bytes <= cap) return ptr;
    if (ptr) cudaFree(ptr);
    ptr = nullptr; cap = 0;
    const size_t want = (bytes + 255) / 256 * 256;
    if (cudaMalloc(&ptr, want) != cudaSuccess) { cudaGetLastError(); ptr = nullptr; return nullptr; }
    cap = want;
    return ptr;
}
void Scratch::release() { if (ptr) cudaFree(ptr); ptr = nullptr; cap = 0; }

// ---- weight cache of the host-pointer entries ---------------------------------
// Keyed by (host pointer, bytes) like the reference's function-local caches; a
// repeated call with the same tensor streams it from HBM, not over PCIe.
const uint8_t* cached_weights(const void* host, size_t bytes) {
    State& s = state();
    auto key = std::make_pair(host, bytes);
    auto it = s.wcache.find(key);
    if (it != s.wcache.end()) return it->second;
    uint8_t* d = nullptr;
    if (cudaMalloc(&d, bytes + 32) != cudaSuccess) { cudaGetLastError(); fail("weight cache: out of device memory (%zu bytes)", bytes); return nullptr; }
    if (cudaMemcpyAsync(d, host, bytes, cudaMemcpyHostToDevice, s.stream) != cudaSuccess) { cudaFree(d); check_launch("weight upload"); return nullptr; }
    cudaMemsetAsync(d + bytes, 0, 32, s.stream);
    s.wcache.emplace(key, d);
    return d;
}

SegTable one_segment(unsigned N) {
    SegTable t;
    std::memset(&t, 0, sizeof t);
    t.nseg = 1; t.row_end[0] = N; t.woff[0] = 0;
    return t;
}

bool make_segments(SegTable& t, unsigned N, const uint64_t* seg_woff, const unsigned* seg_rows, unsigned nseg) {
    if (!seg_woff || !seg_rows || nseg == 0) return fail("segmented gemv: empty segment table");
    if (nseg > (unsigned)kMaxSeg) return fail("segmented gemv: %u segments (at most %d)", nseg, kMaxSeg);
    std::memset(&t, 0, sizeof t);
    unsigned acc = 0;
    for (unsigned i = 0; i < nseg; ++i) { t.yoff[i] = acc; acc += seg_rows[i]; t.row_end[i] = acc; t.woff[i] = seg_woff[i]; }
    t.nseg = nseg;
    if (acc != N) return fail("segmented gemv: segment rows add up to %u, N is %u", acc, N);
    return true;
}

}  // namespace tmc

using namespace tmc;

extern "C" {

bool tm_cuda_init(int device) { return ensure_init(device); }
const char* tm_cuda_last_error(void) { return state().last_error.c_str(); }
unsigned long long tm_cuda_fallback_count(void) { return state().fallbacks; }
unsigned long long tm_cuda_launch_count(void) { return state().launches; }
int tm_cuda_sm_count(void) { return ensure_init(-1) ? state().sm_count : 0; }
unsigned tm_cuda_set_wait_limit_ms(unsigned ms) {
    if (!ensure_init(-1)) return 0;
    State& s = state();
    const unsigned before = (unsigned)(s.wait_limit_ns / 1000000ull);
    if (ms) s.wait_limit_ns = (unsigned long long)ms * 1000000ull;
    return before;
}

size_t tm_cuda_weight_bytes(unsigned dtype, size_t N, size_t K) { return weight_bytes(dtype, N, K); }

// ---- device-pointer kernels ----------------------------------------------------
bool tm_cuda_gemv_q_dev(const float* x, const void* W, float* y, unsigned N, unsigned K, unsigned dtype, void* stream) {
    if (!ensure_init(-1)) return false;
    if (dtype == DT_F16 || dtype == DT_BF16) return launch_gemv_half(x, W, y, N, K, dtype == DT_BF16, (cudaStream_t)stream);
    return launch_gemv(x, (const uint8_t*)W, y, N, K, dtype, one_segment(N), (cudaStream_t)stream);
}

bool tm_cuda_q4_0_from_gguf_dev(void* blocks, size_t nblocks, void* stream) {
    if (!ensure_init(-1)) return false;
    return launch_q4_split_to_interleaved((uint8_t*)blocks, nblocks, (cudaStream_t)stream);
}

bool tm_cuda_gemv_seg_dev(const float* x, const void* W, float* y, unsigned N, unsigned K, unsigned dtype,
                          const uint64_t* seg_woff, const unsigned* seg_rows, unsigned nseg, void* stream) {
    if (!ensure_init(-1)) return false;
    SegTable t;
    if (!make_segments(t, N, seg_woff, seg_rows, nseg)) return false;
    return launch_gemv(x, (const uint8_t*)W, y, N, K, dtype, t, (cudaStream_t)stream);
}

bool tm_cuda_dequant_dev(const void* W, float* out, unsigned N, unsigned K, unsigned dtype, void* stream) {
    if (!ensure_init(-1)) return false;
    return launch_dequant((const uint8_t*)W, out, N, K, dtype, (cudaStream_t)stream);
}

// ---- host-pointer per-tensor entries ---------------------------------------------
bool tm_cuda_gemv_q(const float* x, const void* W, float* y, unsigned N, unsigned K, unsigned dtype) {
    if (!ensure_init(-1)) return false;
    if (!x || !W || !y) return fail("gemv: null pointer");
    const size_t wb = weight_bytes(dtype, N, K);
    if (!wb) return fail("gemv: K=%u is not whole blocks of dtype %u", K, dtype);
    State& s = state();
    const uint8_t* dW = cached_weights(W, wb);
    if (!dW) return false;
    float* dx = (float*)s.io_x.get((size_t)K * 4);
    if (!dx) return fail("gemv: out of device memory");
    // A short y in page-locked host memory is written by the kernel itself (the device sees such memory): that saves
    // the copy back and its DMA latency, a fifth of a small call. Long outputs keep the DMA, which moves them faster
    // than row-by-row stores over PCIe.
    float* dy = nullptr;
    bool direct = false;
    static const unsigned direct_rows = [] { const char* e = std::getenv("TM_DIRECT_Y_ROWS"); return e && *e ? (unsigned)std::atoi(e) : 8192u; }();
    if (N <= direct_rows) {
        cudaPointerAttributes at;
        if (cudaPointerGetAttributes(&at, y) == cudaSuccess && at.type == cudaMemoryTypeHost && at.devicePointer) {
            dy = (float*)at.devicePointer; direct = true;
        } else {
            cudaGetLastError();
        }
    }
    if (!direct) dy = (float*)s.io_y.get((size_t)N * 4);
    if (!dy) return fail("gemv: out of device memory");
    // x in page-locked host memory is not copied by the DMA engine (a dozen microseconds before the kernel can start):
    // the staging kernel reads it over PCIe once, 4 K bytes, and leaves it in the form the GEMV's lanes consume; the GEMV
    // then copies that image instead of staging x in every CTA. Pageable x takes the copy.
    {
        cudaPointerAttributes ax;
        const size_t img = xq_bytes(K, dtype);
        if (img && cudaPointerGetAttributes(&ax, x) == cudaSuccess && ax.type == cudaMemoryTypeHost && ax.devicePointer &&
            (uintptr_t)ax.devicePointer % 16 == 0) {
            uint32_t* xq = (uint32_t*)s.io_xq.get(img);
            if (!xq) return fail("gemv: out of device memory");
            const float* xm = (const float*)ax.devicePointer;
            if (!launch_xprep(xq, xm, nullptr, 0, 0.f, K, dtype, nullptr, s.stream)) return false;
            GemvFuse f{};
            f.xq = xq;
            if (!launch_gemv(xm, dW, dy, N, K, dtype, one_segment(N), s.stream, &f)) return false;
            if (!direct && cudaMemcpyAsync(y, dy, (size_t)N * 4, cudaMemcpyDeviceToHost, s.stream) != cudaSuccess) return check_launch("gemv: y download");
            return sync_stream(s.stream, "gemv");
        }
        cudaGetLastError();
    }
    if (cudaMemcpyAsync(dx, x, (size_t)K * 4, cudaMemcpyHostToDevice, s.stream) != cudaSuccess) return check_launch("gemv: x upload");
    if (!launch_gemv(dx, dW, dy, N, K, dtype, one_segment(N), s.stream)) return false;
    if (!direct && cudaMemcpyAsync(y, dy, (size_t)N * 4, cudaMemcpyDeviceToHost, s.stream) != cudaSuccess) return check_launch("gemv: y download");
    return sync_stream(s.stream, "gemv");
}

bool tm_cuda_q4_gemv(const float* x, const void* Wq, float* y, unsigned N, unsigned K) {
    return tm_cuda_gemv_q(x, Wq, y, N, K, DT_Q4_0);
}

bool tm_cuda_dequant(const void* W, float* out, unsigned N, unsigned K, unsigned dtype) {
    if (!ensure_init(-1)) return false;
    if (!W || !out) return fail("dequant: null pointer");
    const size_t wb = weight_bytes(dtype, N, K);
    if (!wb) return fail("dequant: K=%u is not whole blocks of dtype %u", K, dtype);
    State& s = state();
    const uint8_t* dW = cached_weights(W, wb);
    if (!dW) return false;
    const size_t ob = (size_t)N * K * 4;
    float* dout = (float*)s.io_big.get(ob);
    if (!dout) return fail("dequant: out of device memory (%zu bytes)", ob);
    if (!launch_dequant(dW, dout, N, K, dtype, s.stream)) return false;
    if (cudaMemcpyAsync(out, dout, ob, cudaMemcpyDeviceToHost, s.stream) != cudaSuccess) return check_launch("dequant: download");
    return sync_stream(s.stream, "dequant");
}

size_t tm_cuda_sgemm_q_workspace(unsigned M, unsigned N, unsigned K, unsigned dtype) {
    (void)dtype;
    return gemm_workspace_bytes(M, N, K);
}

bool tm_cuda_sgemm_q_dev(const float* A, const void* W, float* C, unsigned M, unsigned N, unsigned K, unsigned dtype,
                         void* workspace, size_t workspace_bytes, void* stream) {
    if (!ensure_init(-1)) return false;
    return launch_gemm(A, (const uint8_t*)W, C, N, M, N, K, dtype, workspace, workspace_bytes, (cudaStream_t)stream);
}

// Shared body of the host-pointer GEMM entries: nparts tensors against one batch,
// part p filling columns [sum(Ns[0..p)), +Ns[p]) of the M x sum(Ns) result.
static bool gemm_parts_host(const float* A, const void* const* Ws, const unsigned* Ns, unsigned nparts, float* C,
                            unsigned M, unsigned K, unsigned dtype) {
    if (!ensure_init(-1)) return false;
    if (!A || !Ws || !Ns || !C || nparts == 0) return fail("gemm: bad arguments");
    if (M == 0) return fail("gemm: empty batch");
    State& s = state();
    size_t ntot = 0, ws_need = 0;
    for (unsigned p = 0; p < nparts; ++p) {
        if (!Ws[p]) return fail("gemm: null weight pointer");
        if (!weight_bytes(dtype, Ns[p], K)) return fail("gemm: K=%u is not whole blocks of dtype %u", K, dtype);
        ntot += Ns[p];
        ws_need = std::max(ws_need, gemm_workspace_bytes(M, Ns[p], K));
    }
    float* dA = (float*)s.io_a.get((size_t)M * K * 4);
    float* dC = (float*)s.io_big.get((size_t)M * ntot * 4);
    void* ws = s.gemm_ws.get(ws_need);
    if (!dA || !dC || !ws) return fail("gemm: out of device memory");
    if (cudaMemcpyAsync(dA, A, (size_t)M * K * 4, cudaMemcpyHostToDevice, s.stream) != cudaSuccess) return check_launch("gemm: A upload");
    size_t col = 0;
    for (unsigned p = 0; p < nparts; ++p) {
        const uint8_t* dW = cached_weights(Ws[p], weight_bytes(dtype, Ns[p], K));
        if (!dW) return false;
        if (!launch_gemm(dA, dW, dC + col, (unsigned)ntot, M, Ns[p], K, dtype, ws, s.gemm_ws.cap, s.stream)) return false;
        col += Ns[p];
    }
    if (cudaMemcpyAsync(C, dC, (size_t)M * ntot * 4, cudaMemcpyDeviceToHost, s.stream) != cudaSuccess) return check_launch("gemm: C download");
    return sync_stream(s.stream, "gemm");
}

bool tm_cuda_sgemm_q(const float* A, const void* W, float* C, unsigned M, unsigned N, unsigned K, unsigned dtype) {
    return gemm_parts_host(A, &W, &N, 1, C, M, K, dtype);
}
bool tm_cuda_sgemm_q4(const float* A, const void* Wq, float* C, unsigned M, unsigned N, unsigned K) {
    return gemm_parts_host(A, &Wq, &N, 1, C, M, K, DT_Q4_0);
}
bool tm_cuda_q4_prefill(const float* A, const void* const* Wqs, const unsigned* Ns, unsigned nparts, float* C,
                        unsigned M, unsigned K) {
    return gemm_parts_host(A, Wqs, Ns, nparts, C, M, K, DT_Q4_0);
}

size_t tm_cuda_trace_read(unsigned long long* out, size_t cap_launches) {
    State& s = state();
    if (!s.ready || !s.trace_dev || !out) return 0;
    cudaStreamSynchronize(s.stream);
    unsigned long long n = 0;
    if (cudaMemcpy(&n, s.trace_dev, 8, cudaMemcpyDeviceToHost) != cudaSuccess) { check_launch("trace_read"); return 0; }
    if (n > (unsigned long long)kTraceLaunches) n = kTraceLaunches;
    if (n > cap_launches) n = cap_launches;
    if (n && cudaMemcpy(out, s.trace_dev + 1, n * kTraceWords * 8, cudaMemcpyDeviceToHost) != cudaSuccess) { check_launch("trace_read"); return 0; }
    cudaMemset(s.trace_dev, 0, 8);
    return (size_t)n;
}

void tm_cuda_release_weights(void) {
    State& s = state();
    if (!s.ready) return;
    cudaStreamSynchronize(s.stream);
    for (auto& kv : s.wcache) cudaFree(kv.second);
    s.wcache.clear();
    // the lane's registrations are keyed by host address too: graphs first (they hold the device pointers)
    tm_cuda_tok_graph_destroy(-1);
    for (WeightBuf& w : s.wbufs) if (w.ptr) { cudaFree(w.ptr); w.ptr = nullptr; w.bytes = 0; }
    s.wreg.clear();
    s.shared_base = nullptr; s.shared_id = -1;
    for (auto& kv : s.norm_w) cudaFree(kv.second);
    s.norm_w.clear();
    s.x_prep.stamp = ~0ull;                               // the staged x image named norm weights that are gone
}

// ---- the reference's symbol names ----------------------------------------------
// An unmodified caller declares these weak (tensormark/llama.h:35-152) and tests them
// for null; exporting them makes this library the backend it finds.
bool tm_metal_q4_gemv(const float* x, const void* Wq, float* y, unsigned N, unsigned K) { return tm_cuda_q4_gemv(x, Wq, y, N, K); }
bool tm_metal_sgemm_q4(const float* A, const void* Wq, float* C, unsigned M, unsigned N, unsigned K) { return tm_cuda_sgemm_q4(A, Wq, C, M, N, K); }
bool tm_metal_q4_prefill(const float* A, const void* const* Wqs, const unsigned* Ns, unsigned nparts, float* C, unsigned M, unsigned K) {
    return tm_cuda_q4_prefill(A, Wqs, Ns, nparts, C, M, K);
}

}  // extern "C"
