// include/gemv_pool.h — row-chunk worker pool for CPU GEMV kernels.
//
// Host-side mirror of the reference's fixed-purpose pool (tensormark/gemv_pool.h):
// same job description (GemvArgs 41-50, GemvJob 69-73), same claim protocol
// (run_slices 253-264: 64-row chunks taken from an atomic counter, the caller takes
// part, kernels receive GLOBAL row bounds and the BASE output pointer) and the same
// dispatch() validation (296-315). The reference builds only on macOS/Windows
// (tm_host.h:21-23); this one is portable C++ over std::thread, sized by
// TM_THREADS or the hardware thread count. On this path it threads the CPU side
// of a comparison (dequantize + dot); the GPU path never goes through it.
#pragma once

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstdlib>
#include <mutex>
#include <span>
#include <stdexcept>
#include <thread>
#include <vector>

namespace tmllama {

struct GemvArgs {
    const void* w = nullptr;
    std::span<const float> x{};
    std::span<const std::int8_t> xq{};   // int8 activations (unused by the fp32 kernels)
    std::span<const float> xs{};         // per-32-block activation scales
    std::span<const std::int8_t> xd{};   // deinterleaved int8 activations
    std::span<float> y{};                // BASE of the output: kernels index global rows
    int n_in = 0;
};

#ifndef TM_GEMV_CHUNK
#define TM_GEMV_CHUNK 64
#endif

struct GemvJob {
    void (*kern)(const GemvArgs&, int o0, int o1) = nullptr;
    GemvArgs a{};
    int n_out = 0, chunk = TM_GEMV_CHUNK;
};

class GemvPool {
public:
    explicit GemvPool(int requested_threads = 0) {
        int n = requested_threads;
        if (n <= 0) {
            if (const char* e = std::getenv("TM_THREADS")) n = std::atoi(e);
        }
        if (n <= 0) n = (int)std::thread::hardware_concurrency();
        if (n <= 0) n = 1;
        nthreads = n;
        workers_.reserve((size_t)n - 1);
        for (int i = 1; i < n; ++i) workers_.emplace_back([this] { worker(); });
    }
    GemvPool(const GemvPool&) = delete;
    GemvPool& operator=(const GemvPool&) = delete;
    ~GemvPool() {
        {
            std::lock_guard<std::mutex> lk(mu_);
            stopping_ = true;
        }
        start_cv_.notify_all();
        for (auto& t : workers_) t.join();
    }

    int nthreads = 1;   // includes the calling thread

    // Claim chunks until the rows run out. Kernels get global [o0, o1) and index
    // j.a.y from its base (adding o0 again would write past the tensor).
    void run_slices(const GemvJob& j) {
        for (;;) {
            const std::uint64_t start = next_.fetch_add(1, std::memory_order_relaxed) * (std::uint64_t)j.chunk;
            if (start >= (std::uint64_t)j.n_out) return;
            const std::uint64_t end = std::min<std::uint64_t>(start + (std::uint64_t)j.chunk, (std::uint64_t)j.n_out);
            j.kern(j.a, (int)start, (int)end);
        }
    }

    // One job at a time; returns when every row has been computed.
    void dispatch(const GemvJob& j) {
        if (!j.kern || j.chunk <= 0 || j.a.n_in < 0 || j.n_out < 0) throw std::invalid_argument("invalid GEMV job");
        std::lock_guard<std::mutex> whole(dispatch_mu_);
        {
            std::lock_guard<std::mutex> lk(mu_);
            job_ = j;
            next_.store(0, std::memory_order_relaxed);
            done_.store(0, std::memory_order_relaxed);
            ++gen_;
        }
        start_cv_.notify_all();
        run_slices(j);
        std::unique_lock<std::mutex> lk(mu_);
        done_cv_.wait(lk, [&] { return done_.load(std::memory_order_acquire) == nthreads - 1; });
    }

private:
    void worker() {
        std::uint64_t seen = 0;
        for (;;) {
            GemvJob j;
            {
                std::unique_lock<std::mutex> lk(mu_);
                start_cv_.wait(lk, [&] { return stopping_ || gen_ != seen; });
                if (stopping_) return;
                seen = gen_;
                j = job_;
            }
            run_slices(j);
            {
                std::lock_guard<std::mutex> lk(mu_);
                done_.fetch_add(1, std::memory_order_release);
            }
            done_cv_.notify_one();
        }
    }

    GemvJob job_{};
    std::atomic<std::uint64_t> next_{0};
    std::atomic<int> done_{0};
    std::uint64_t gen_ = 0;
    bool stopping_ = false;
    std::mutex mu_, dispatch_mu_;
    std::condition_variable start_cv_, done_cv_;
    std::vector<std::thread> workers_;
};

// Process-wide pool, created on first use and never destroyed.
inline GemvPool& gemv_pool() {
    static GemvPool* p = new GemvPool();
    return *p;
}

}  // namespace tmllama
