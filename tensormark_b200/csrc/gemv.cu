// gemv.cu — streaming block-quantized GEMV for sm_100a:  y[N] = W[N x K] * x[K].
//
// Replaces the cooperative-row Metal GEMVs (tensormark/metal.h:359-440 Q4_0,
// 641-679 Q4_1, 708-754 Q5_K, 775-822 Q6_K, and their segmented forms 511-567,
// 915-1078) and adds the Q8_0 kernel the reference GPU lane lacks.
//
// The kernel is bound by HBM: every weight byte is read exactly once, at its
// serialized width. Structure:
//   * Each warp owns a private ring of STAGES shared-memory stages and streams its
//     rows through it with bulk asynchronous copies (cp.async.bulk global ->
//     shared, completion on an mbarrier). One elected lane issues the copies; no
//     thread ever holds a weight load in a register scoreboard, so the bytes in
//     flight per SM are set by the ring size, not by occupancy.
//   * A warp task is a group of R consecutive rows times one step of the row
//     (2048 or 1024 weights); the lane's activations for that step are loaded into
//     registers once and reused for the R rows.
//   * x is staged once per CTA into shared memory as block floating point (a scale and
//     three int8 planes per 32 activations, see gemv_lanes.cuh) in the byte layout
//     the lanes consume, together with the plain fp32 sums that carry zero points
//     and mins; the inner loop is then integer dot products (dp4a) on the code bytes.
//   * Rows are summed over lanes with shuffles in a fixed order, so a row's
//     result does not depend on the grid, on R, or on whether it was reached
//     through a segment table: the segmented launch is bit-identical to separate
//     launches (the property tensormark/metal.h:504-510 requires).
//   * The weight prefetch is issued before griddepcontrol.wait, so under
//     programmatic dependent launch a GEMV starts pulling its weights while the
//     kernel that produces its x is still running.
//
// Fast-path requirement: every row starts on a 16-byte boundary (W, segment
// offsets and row_bytes multiples of 16). Anything else takes gemv_generic, a
// plain byte-granular kernel with the same per-row arithmetic contract
// (tolerance-level, not bitwise, agreement with the fast path).
#include "common.cuh"
#include "gemv_lanes.cuh"
#include "exchange.cuh"

#include <cstdlib>

namespace tmc {

namespace {

constexpr int kMaxWarps = 16;       // warps per CTA: 16 (512 threads x 128 registers fill the register file) or 8
constexpr int kMaxStages = 8;      // ring depth per warp is chosen at launch, 2..kMaxStages

struct GemvParams {
    const uint8_t* W;
    const float* x;
    float* y;
    uint32_t N, K, row_bytes;
    uint32_t stages, rows_per_cta;
    // optional fusions (decode chain): a transform of x while it is staged, and y += instead of y =
    const float* x2;            // x_op 1: rmsnorm weights; x_op 2: the "up" vector
    float eps;
    uint32_t x_op;              // 0 plain, 1 x*rsqrt(mean(x^2)+eps)*x2, 2 silu(x)*x2
    uint32_t accumulate;
    SegTable seg;
    Exchange xc;                // row-sharded models: wait for peers before x, push y to peers after
    unsigned long long* trace;  // kernel timeline, nullptr when off
    int* status;
    // x already in the lanes' unit form (written once per launch by xprep_kernel): the CTA bulk-copies the image
    // instead of staging x itself. Layout: 16 header words ([0] = the RMSNorm
    // factor as a float, 1.0 when none), then the units.
    const uint32_t* xq;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// One probe that never suspends the thread: a third of try_wait's latency when the phase is already complete.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false when the time limit ran out (the caller records it and leaves).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned long long limit_ns = kWaitLimitNs) {
    if (mbar_test(bar, parity)) return true;
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_ns() - t0 > limit_ns) return false;
    }
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// ---- thread-block clusters: the CTAs of a cluster share the staging of x ---------------------
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_size() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// The address of this CTA's shared-memory object `p` in CTA `rank` of the cluster (generic pointer).
template <typename T> __device__ __forceinline__ T* cluster_map(T* p, uint32_t rank) {
    uint64_t out;
    asm volatile("mapa.u64 %0, %1, %2;" : "=l"(out) : "l"((uint64_t)(uintptr_t)p), "r"(rank));
    return (T*)(uintptr_t)out;
}

__device__ __forceinline__ const uint8_t* row_ptr(const GemvParams& p, uint32_t row) {
    uint32_t s = 0, start = 0;
    while (s + 1 < p.seg.nseg && row >= p.seg.row_end[s]) { start = p.seg.row_end[s]; ++s; }
    return p.W + p.seg.woff[s] + (size_t)(row - start) * p.row_bytes;
}

// Element of y that receives `row` (segments may land at separate offsets of y).
__device__ __forceinline__ uint32_t y_index(const GemvParams& p, uint32_t row) {
    uint32_t s = 0, start = 0;
    while (s + 1 < p.seg.nseg && row >= p.seg.row_end[s]) { start = p.seg.row_end[s]; ++s; }
    return p.seg.yoff[s] + (row - start);
}

// Store one finished row: here and, for a sharded model, into every peer's copy of y.
__device__ __forceinline__ void store_row(const GemvParams& p, uint32_t e, float v) {
    p.y[e] = v;
    for (uint32_t q = 0; q < p.xc.npush; ++q) p.xc.peer_y[q][e] = v;
}

template <int DT> __device__ __forceinline__ int lane_valid(int lane, int units_in_chunk) {
    using L = Lane<DT>;
    if constexpr (L::LANE_UNITS == 2) {
        const int v = units_in_chunk - 2 * lane;
        return v < 0 ? 0 : (v > 2 ? 2 : v);
    } else {
        return units_in_chunk;      // K-quant lanes test their own super-block index against it
    }
}


// ---- staging of x: block floating point planes in the lanes' byte layout -------
// Eight lanes per 32-block, four activations (one float4) per lane: the block maximum and the run sums come from
// three shuffle stages, the plane bytes leave as packed stores. A warp stages eight blocks (256 activations, one
// "group") per pass; it takes groups g_first, g_first + g_step, ... below g_end. `units` is shared memory (a CTA
// staging for itself) or global memory (staging once for every CTA of a later launch). Returns this lane's share
// of sum(x^2) for x_op 1 (RMSNorm: x * w is staged, the factor rsqrt(mean(x^2) + eps) is one number for the whole
// vector and multiplies the finished row sums instead); x_op 2 stages silu(x) * x2.
template <int DT>
__device__ __forceinline__ float stage_groups(uint32_t* units, const float* x, const float* x2, uint32_t x_op, uint32_t K,
                                              uint32_t g_first, uint32_t g_end, uint32_t g_step, int lane) {
    using L = Lane<DT>;
    constexpr int B = 2;
    const uint32_t nblk = K / 32, li = lane & 7u, sub = lane >> 3;
    const float4* xg4 = reinterpret_cast<const float4*>(x);
    const float4* x24 = reinterpret_cast<const float4*>(x2);
    float ss = 0.f;
    // The loads of the next group are issued before the current group is quantized: a warp's passes are
    // otherwise a chain of L2 latencies.
    float4 nv[B], nw[B];
    auto fetch = [&](uint32_t g) {
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const uint32_t b = g * (4 * B) + 4 * j + sub;
            const bool in = g < g_end && b < nblk;
            nv[j] = in ? __ldcg(xg4 + b * 8 + li) : make_float4(0.f, 0.f, 0.f, 0.f);
            nw[j] = (in && x_op != 0u) ? __ldcg(x24 + b * 8 + li) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    fetch(g_first);
    for (uint32_t g = g_first; g < g_end; g += g_step) {
        const uint32_t b0 = g * (4 * B);
        float4 v[B];
        float am[B], s8[B], s16[B], s32[B];
        bool bad[B];
        float4 w2s[B];
#pragma unroll
        for (int j = 0; j < B; ++j) { v[j] = nv[j]; w2s[j] = nw[j]; }
        fetch(g + g_step);
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const uint32_t b = b0 + 4 * j + sub;
            if (x_op != 0u && b < nblk) {
                const float4 w2 = w2s[j];
                if (x_op == 1u) {
                    ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss); ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
                    v[j].x *= w2.x; v[j].y *= w2.y; v[j].z *= w2.z; v[j].w *= w2.w;
                } else {
                    // silu(x) * up with the hardware exponential and reciprocal: relative error 2^-21, inside what the
                    // fixed-point planes that follow keep
                    v[j].x = __fdividef(v[j].x, 1.0f + __expf(-v[j].x)) * w2.x; v[j].y = __fdividef(v[j].y, 1.0f + __expf(-v[j].y)) * w2.y;
                    v[j].z = __fdividef(v[j].z, 1.0f + __expf(-v[j].z)) * w2.z; v[j].w = __fdividef(v[j].w, 1.0f + __expf(-v[j].w)) * w2.w;
                }
            }
            am[j] = fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w)));
            const float any_nan = (v[j].x + v[j].y) + (v[j].z + v[j].w);         // NaN if any element is NaN
            bad[j] = !(am[j] <= 3.0e38f) || any_nan != any_nan;
            s8[j] = (v[j].x + v[j].y) + (v[j].z + v[j].w);
        }
#pragma unroll
        for (int o = 1; o <= 4; o <<= 1)
#pragma unroll
            for (int j = 0; j < B; ++j) {
                am[j] = fmaxf(am[j], __shfl_xor_sync(0xffffffffu, am[j], o));
                bad[j] = bad[j] || __shfl_xor_sync(0xffffffffu, (int)bad[j], o);
            }
        if (L::NEEDS_SUMS) {
#pragma unroll
            for (int j = 0; j < B; ++j) {
                s8[j] += __shfl_xor_sync(0xffffffffu, s8[j], 1);                  // 8 activations
                s16[j] = s8[j] + __shfl_xor_sync(0xffffffffu, s8[j], 2);          // 16
                s32[j] = s16[j] + __shfl_xor_sync(0xffffffffu, s16[j], 4);        // 32
            }
        } else {
#pragma unroll
            for (int j = 0; j < B; ++j) s16[j] = s32[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const uint32_t b = b0 + 4 * j + sub;
            if (b < nblk) {
                float inv;
                const float sc = block_scale(am[j], bad[j], inv);
                int8_t q0[kPlanes], q1[kPlanes], q2[kPlanes], q3[kPlanes];
                quantize_elem(v[j].x, inv, q0); quantize_elem(v[j].y, inv, q1);
                quantize_elem(v[j].z, inv, q2); quantize_elem(v[j].w, inv, q3);
#pragma unroll
                for (int t = 0; t < kPlanes; ++t)
                    L::store_quad(units, b * 32 + 4 * li, t,
                                  (uint32_t)(uint8_t)q0[t] | ((uint32_t)(uint8_t)q1[t] << 8) |
                                  ((uint32_t)(uint8_t)q2[t] << 16) | ((uint32_t)(uint8_t)q3[t] << 24));
                L::scalars(units, b, (int)(4 * li), (int)li, sc, s8[j], s16[j], s32[j]);
            }
        }
    }
    return ss;
}

// One CTA stages the whole vector x (K activations) for a consumer of format CDT into `out` (global memory: 16 header
// words, then the units), and writes the RMSNorm factor into out[0]. Warp w takes groups w, w + nwarps, ... so the
// sum of squares is added in the same order as when a GEMV CTA stages x for itself.
template <int CDT>
__device__ __forceinline__ void stage_vector(uint32_t* out, const float* x, const float* x2, uint32_t x_op, float eps, uint32_t K, float* red) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const uint32_t ngroups = (K + 255u) / 256u;
    float ss = stage_groups<CDT>(out + kXqHeaderWords, x, x2, x_op, K, (uint32_t)warp, ngroups, (uint32_t)nwarps, lane);
    if (x_op == 1u) {
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        if (threadIdx.x == 0) {
            float tot = 0.f;
            for (int w = 0; w < nwarps; ++w) tot += red[w];
            out[0] = __float_as_uint(1.0f / sqrtf(tot / (float)K + eps));
        }
    } else if (threadIdx.x == 0) {
        out[0] = __float_as_uint(1.0f);
    }
}
// x in unit form, once per launch. RMSNorm needs the
// sum over the whole vector and runs as ONE CTA of 16 warps; the other transforms have no cross-group term and run
// as many small CTAs as there are groups to cover.
template <int CDT>
__global__ void __launch_bounds__(512) xprep_kernel(uint32_t* out, const float* x, const float* x2, uint32_t x_op, float eps, uint32_t K,
                                                    const Exchange xc, int* status) {
    __shared__ float red[16];
    // The GEMV that follows may become resident and prefetch its weights at once; it waits for this grid itself.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (x_op == 1u)                                        // norm weights: static, and out of L2 since the last token
        for (uint32_t i = (blockIdx.x * blockDim.x + threadIdx.x) * 32u; i < K; i += gridDim.x * blockDim.x * 32u)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(x2 + i) : "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    exchange_wait(xc, status);
    if (gridDim.x == 1) { stage_vector<CDT>(out, x, x2, x_op, eps, K, red); return; }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const uint32_t ngroups = (K + 255u) / 256u, g = blockIdx.x * nwarps + warp;
    if (g < ngroups) (void)stage_groups<CDT>(out + kXqHeaderWords, x, x2, x_op, K, g, g + 1, 1u, lane);
    if (blockIdx.x == 0 && threadIdx.x == 0) out[0] = __float_as_uint(1.0f);
}

// Shared memory: [x units: one per lane and step][mbarriers][stages]
//
// Work split: the rows are cut into one contiguous range per CTA (rows_per_cta =
// ceil(N / grid)). Inside a CTA the warps form teams of `nchunks` warps, one warp per step of
// the row: a warp keeps the activations of ITS step in registers for the whole kernel and
// streams that step of the team's rows, R rows per ring item; teams take the CTA's row groups
// round-robin. With one step per row (K <= 2048) every warp is its own team and stores y
// directly; with several steps the warps leave per-step partial sums in shared memory and the
// CTA adds them in step order after one barrier. Which mode runs depends on K only, never on
// N, so a row's bits are the same in a segmented and in a separate launch.
template <int DT, int R, int kWarps>
__global__ void __launch_bounds__(kWarps * 32, 16 / kWarps) gemv_stream(const GemvParams p) {
    using L = Lane<DT>;
    constexpr int ROWCAP = L::STEP_BYTES;                  // multiple of 16
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned long long* tr = nullptr;                       // this launch's timeline record (CTA 0, thread 0 only)
    if (p.trace && blockIdx.x == 0 && threadIdx.x == 0) {
        const unsigned long long slot = atomicAdd(p.trace, 1ull);
        if (slot < (unsigned long long)kTraceLaunches) {
            tr = p.trace + 1 + slot * kTraceWords;
            tr[0] = global_ns();
            tr[4] = ((unsigned long long)p.N << 32) | p.K;
            tr[5] = (unsigned long long)DT | ((unsigned long long)p.x_op << 8) | ((unsigned long long)kWarps << 16) | ((unsigned long long)R << 24);
        }
    }
    const uint32_t nchunks = (p.K + L::STEP_W - 1) / L::STEP_W;
    const uint32_t nunits = nchunks * 32u;
    uint32_t* units = reinterpret_cast<uint32_t*>(smem);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (((size_t)nunits * L::XW * 4 + 127) / 128) * 128);
    const uint32_t S = p.stages;
    uint8_t* stages = reinterpret_cast<uint8_t*>(bars) + ((kMaxWarps * kMaxStages * 8 + 127) / 128) * 128;
    uint64_t* mybar = bars + warp * kMaxStages;
    uint8_t* mystage = stages + (size_t)warp * S * R * ROWCAP;

    float* partial = reinterpret_cast<float*>(stages + (size_t)kWarps * S * R * ROWCAP);   // [rows_per_cta][nchunks], only when nchunks > 1

    const uint32_t teams = kWarps / nchunks;               // >= 1 (the launcher guarantees nchunks <= kWarps)
    const uint32_t team = (uint32_t)warp / nchunks, myc = (uint32_t)warp % nchunks;
    const uint32_t cta_lo = min(p.N, blockIdx.x * p.rows_per_cta), cta_hi = min(p.N, cta_lo + p.rows_per_cta);
    const uint32_t row_first = cta_lo + team * R, grp_stride = teams * R;
    const uint32_t items = (team < teams && row_first < cta_hi) ? (cta_hi - row_first + grp_stride - 1) / grp_stride : 0;

    if (lane == 0) {
        for (uint32_t s = 0; s < S; ++s) mbar_init(&mybar[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    const uint32_t csize = cluster_size(), crank = csize > 1 ? cluster_rank() : 0u;
    if (csize > 1) cluster_arrive();                        // "this CTA runs": awaited before the first access to a peer's shared memory

    // Issue cursor (same value in every lane): next item = rows [irow, irow+R) x this warp's step.
    const uint32_t off = myc * (uint32_t)L::STEP_BYTES;
    const uint32_t bytes = p.row_bytes > off ? min((uint32_t)L::STEP_BYTES, p.row_bytes - off) : 0u;
    uint32_t irow = row_first, issued = 0;
    auto issue = [&](uint32_t slot) {
        const uint32_t rows = min((uint32_t)R, cta_hi - irow);
        if (lane == 0) mbar_expect_tx(&mybar[slot], rows * bytes);
        if ((uint32_t)lane < rows)                          // one row copy per lane, issued in parallel
            bulk_g2s(mystage + ((size_t)slot * R + lane) * ROWCAP, row_ptr(p, irow + lane) + off, bytes, &mybar[slot]);
        irow += grp_stride;
        ++issued;
    };
    for (uint32_t s = 0; s < S && issued < items; ++s) issue(s);

    // RMSNorm weights are read once per token, 4 GB of streamed blocks apart: by then they have left L2, and their DRAM
    // latency (1.1-1.5 us, measured as the difference of the x phase with and without these loads) would sit between
    // the dependency wait and the first row. They do not depend on the preceding kernel: ask for them now.
    if (p.x_op == 1u && !p.xq) {
        for (uint32_t i = threadIdx.x * 32u; i < p.K; i += blockDim.x * 32u)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.x2 + i) : "memory");
    }
    // x itself may still be written by the preceding kernel, but L2 is where its writes land: asking for the lines now
    // costs nothing when they are there and saves the DRAM round trip after the wait when they are not (an activation
    // vector that was last touched a few hundred MB of weights ago).
    if (!p.xq) {
        for (uint32_t i = threadIdx.x * 32u; i < p.K; i += blockDim.x * 32u)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.x + i) : "memory");
    }
    // Everything above touches only weights. x may be written by the preceding
    // kernel in the stream: wait for it here, and let the next kernel start its own
    // weight prefetch.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    exchange_wait(p.xc, p.status);                          // sharded models: x is complete once every peer has pushed
    if (tr) tr[1] = global_ns();

    // ---- x units into shared memory --------------------------------------------
    // Either the image was written once for the whole launch (p.xq: one bulk copy per CTA), or this CTA stages x
    // itself. Every CTA needs all of x, and staging it costs as much as streaming a few hundred KB of weights, so the
    // CTAs of a cluster share the work: CTA r of C stages groups [r*gpc, (r+1)*gpc) into ITS shared memory, and after
    // the cluster barrier every warp reads its unit from the CTA that staged it (distributed shared memory). A launch
    // without clusters is the case C = 1.
    const uint32_t ngroups = (p.K + 255u) / 256u, gpc = (ngroups + csize - 1) / csize;
    const uint32_t g_lo = min(ngroups, crank * gpc), g_hi = min(ngroups, g_lo + gpc);
    __shared__ float xsum[8];                               // RMSNorm: one partial sum of squares per CTA of the cluster
    __shared__ float red[kWarps];
    __shared__ __align__(8) uint64_t xbar;
    float xq_norm = 1.f;
    if (p.xq) {
        const uint32_t xbytes = nunits * (uint32_t)L::XW * 4u;
        if (threadIdx.x == 0) {
            mbar_init(&xbar, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            mbar_expect_tx(&xbar, xbytes);
            bulk_g2s(units, p.xq + kXqHeaderWords, xbytes, &xbar);
            xq_norm = __uint_as_float(__ldcg(p.xq));
            if (!mbar_wait(&xbar, 0)) *(volatile int*)p.status = 1;
            red[0] = xq_norm;
        }
    } else {
        float ss = stage_groups<DT>(units, p.x, p.x2, p.x_op, p.K, g_lo + (uint32_t)warp, g_hi, (uint32_t)kWarps, lane);
        if (p.x_op == 1u) {
            // this CTA's share of sum(x^2), handed to every CTA of the cluster below
#pragma unroll
            for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) red[warp] = ss;
        }
    }
    if (csize > 1) {
        cluster_wait();                                     // every CTA of the cluster has started
        if (p.x_op == 1u) {
            __syncthreads();
            if (threadIdx.x < csize) {
                float tot = 0.f;
#pragma unroll
                for (int w = 0; w < kWarps; ++w) tot += red[w];
                *cluster_map(&xsum[crank], threadIdx.x) = tot;
            }
        }
        cluster_arrive();                                   // x units and partial sums are in place ...
        cluster_wait();                                     // ... in every CTA
    } else {
        __syncthreads();                                    // x units and the warps' partial sums of squares are in place
    }
    float norm_inv = 1.f;
    if (p.xq) {
        norm_inv = red[0];                                  // written with the units by whoever staged them
    } else if (p.x_op == 1u) {
        // every thread adds the partial sums itself (broadcast reads, fixed order): no second barrier
        float tot = 0.f;
        if (csize > 1) {
            for (uint32_t c = 0; c < csize; ++c) tot += xsum[c];
        } else {
#pragma unroll
            for (int w = 0; w < kWarps; ++w) tot += red[w];
        }
        norm_inv = 1.0f / sqrtf(tot / (float)p.K + p.eps);
    }
    if (tr) tr[2] = global_ns();

    // ---- consume -------------------------------------------------------------
    typename L::X xr;
    bool dead = false;
    uint32_t slot = 0, phase = 0, row0 = row_first;
    if (items) {
        const uint32_t u = myc * 32u + (uint32_t)lane;
        constexpr uint32_t kUnitsPerGroup = 256u * 32u / (uint32_t)L::STEP_W;
        const uint32_t owner = min(csize - 1u, (u / kUnitsPerGroup) / gpc);
        load_x_unit<DT>(xr, csize > 1 ? cluster_map(units, owner) : units, u);
    }
    if (csize > 1) cluster_arrive();                        // this CTA is done with its peers' shared memory
    const uint32_t wchunk = min((uint32_t)L::STEP_W, p.K - myc * L::STEP_W);
    const int valid = lane_valid<DT>(lane, (int)(wchunk / L::UNIT_W));
    const bool full_chunk = wchunk == (uint32_t)L::STEP_W;  // every lane then has all of its units
    bool landed = false;                                    // the probe of this item's stage, made while the previous item was summed
    for (uint32_t t = 0; t < items; ++t) {
        float acc[R];
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = 0.f;
        if (!landed && !mbar_wait(&mybar[slot], phase)) { dead = true; break; }
        const uint8_t* st = mystage + (size_t)slot * R * ROWCAP;
        const uint32_t rows = min((uint32_t)R, cta_hi - row0);
        if (full_chunk && rows == (uint32_t)R) {
            // the common item - R rows of a whole step - without the per-row and per-block tests (both warp-uniform
            // here, but a branch each in the general form below); same arithmetic, same bits
#pragma unroll
            for (int r = 0; r < R; ++r)
                acc[r] = L::dot(st + r * ROWCAP + (L::LANE_UNITS == 2 ? lane * L::LANE_BYTES : 0), xr, lane, L::LANE_UNITS == 2 ? 2 : L::STEP_W / L::UNIT_W);
        } else if (L::LANE_UNITS == 2 ? valid > 0 : true) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                if ((uint32_t)r < rows) {                   // warp-uniform: rows past the range were never copied
                    const uint8_t* rowp = st + r * ROWCAP + (L::LANE_UNITS == 2 ? lane * L::LANE_BYTES : 0);
                    acc[r] = L::dot(rowp, xr, lane, valid);
                }
            }
        }
        __syncwarp();                                       // every lane is done with this stage
        if (issued < items) issue(slot);
        if (++slot == S) { slot = 0; phase ^= 1u; }
        landed = t + 1 < items && mbar_test(&mybar[slot], phase);
        // Sum over lanes. The butterfly order (xor 16, 8, 4, 2, 1) is the same for every R, so a
        // row's bits do not depend on how rows were grouped; with R > 1 the first stages also
        // fold the R rows onto disjoint lanes to save shuffles.
        float v;
        int my_row;
        if constexpr (R == 4) {
            const bool h16 = lane & 16, h8 = lane & 8;
            float k0 = h16 ? acc[2] : acc[0], k1 = h16 ? acc[3] : acc[1];
            const float s0 = h16 ? acc[0] : acc[2], s1 = h16 ? acc[1] : acc[3];
            k0 += __shfl_xor_sync(0xffffffffu, s0, 16);
            k1 += __shfl_xor_sync(0xffffffffu, s1, 16);
            v = h8 ? k1 : k0;
            const float sv = h8 ? k0 : k1;
            v += __shfl_xor_sync(0xffffffffu, sv, 8);
            my_row = (h16 ? 2 : 0) + (h8 ? 1 : 0);
        } else if constexpr (R == 2) {
            const bool h16 = lane & 16;
            v = h16 ? acc[1] : acc[0];
            const float sv = h16 ? acc[0] : acc[1];
            v += __shfl_xor_sync(0xffffffffu, sv, 16);
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            my_row = h16 ? 1 : 0;
        } else {
            v = acc[0];
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            my_row = 0;
        }
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        if ((lane & 7) == 0 && (R == 4 || (lane & 8) == 0) && (uint32_t)my_row < rows) {
            const uint32_t row = row0 + (uint32_t)my_row;
            if (nchunks == 1) {
                const uint32_t e = y_index(p, row);
                if (p.x_op == 1u) v *= norm_inv;
                if (p.accumulate) v += p.y[e];              // residual add folded into the store
                store_row(p, e, v);
            } else {
                partial[(size_t)(row - cta_lo) * nchunks + myc] = v;
            }
        }
        row0 += grp_stride;
    }
    if (nchunks > 1) {
        // every step's partial sum of every row of this CTA is in shared memory: add them in step order
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < cta_hi - cta_lo; i += blockDim.x) {
            float v = partial[(size_t)i * nchunks];
            for (uint32_t cc = 1; cc < nchunks; ++cc) v += partial[(size_t)i * nchunks + cc];
            const uint32_t e = y_index(p, cta_lo + i);
            if (p.x_op == 1u) v *= norm_inv;
            if (p.accumulate) v += p.y[e];
            store_row(p, e, v);
        }
    }
    exchange_signal(p.xc);                                  // sharded models: this CTA's rows are on every peer
    if (tr) tr[3] = global_ns();
    if (csize > 1) cluster_wait();                          // no CTA leaves while a peer may still read its x units
    if (dead) {
        // A copy never completed. Record it, give the copies still in flight a last
        // bounded chance to land (they target this CTA's shared memory) and leave.
        if (lane == 0) {
            *(volatile int*)p.status = 1;
            for (uint32_t s = 0; s < S; ++s) (void)mbar_wait(&mybar[s], 0, 50000000ull), (void)mbar_wait(&mybar[s], 1, 50000000ull);
        }
    }
}

// ---- generic kernel: any alignment, byte loads, one warp per row --------------
template <int DT>
__device__ float generic_row(const uint8_t* r, const float* x, uint32_t K, int lane);

__device__ __forceinline__ float ldh(const uint8_t* p) { return half_to_float((uint32_t)p[0] | ((uint32_t)p[1] << 8)); }

template <> __device__ float generic_row<1>(const uint8_t* r, const float* x, uint32_t K, int lane) {
    float acc = 0.f;
    for (uint32_t b = lane; b < K / 32; b += 32) {
        const uint8_t* q = r + (size_t)b * 18;
        float s = 0.f;
        for (int j = 0; j < 16; ++j)
            s += (float)((int)(q[2 + j] & 15) - 8) * x[b * 32 + 2 * j] + (float)((int)(q[2 + j] >> 4) - 8) * x[b * 32 + 2 * j + 1];
        acc += s * ldh(q);
    }
    return acc;
}
template <> __device__ float generic_row<9>(const uint8_t* r, const float* x, uint32_t K, int lane) {
    float acc = 0.f;
    for (uint32_t b = lane; b < K / 32; b += 32) {
        const uint8_t* q = r + (size_t)b * 18;
        float s = 0.f;
        for (int j = 0; j < 16; ++j)
            s += (float)((int)(q[2 + j] & 15) - 8) * x[b * 32 + j] + (float)((int)(q[2 + j] >> 4) - 8) * x[b * 32 + 16 + j];
        acc += s * ldh(q);
    }
    return acc;
}
// TQ2: the reference's code-counting dot (quant.h:520-531): with lo / hi the two bits of a code,
// sum w x = d * (sum_{lo} x + 2 sum_{hi} x - sum x) per 128-block; one block per lane iteration.
template <> __device__ float generic_row<7>(const uint8_t* r, const float* x, uint32_t K, int lane) {
    float acc = 0.f;
    for (uint32_t b = lane; b < K / 128; b += 32) {
        const uint8_t* q = r + (size_t)b * 34;
        float lo = 0.f, hi = 0.f, all = 0.f;
        for (int j = 0; j < 32; ++j) {
            const uint32_t byte = q[2 + j];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const float xv = x[b * 128 + 4 * j + t];
                const uint32_t c = (byte >> (2 * t)) & 3u;
                all += xv;
                if (c & 1u) lo += xv;
                if (c & 2u) hi += xv;
            }
        }
        acc += ldh(q) * (lo + 2.f * hi - all);
    }
    return acc;
}
template <> __device__ float generic_row<0>(const uint8_t* r, const float* x, uint32_t K, int lane) {
    float acc = 0.f;
    for (uint32_t b = lane; b < K / 32; b += 32) {
        const uint8_t* q = r + (size_t)b * 34;
        float s = 0.f;
        for (int j = 0; j < 32; ++j) s += (float)(int8_t)q[2 + j] * x[b * 32 + j];
        acc += s * ldh(q);
    }
    return acc;
}
template <> __device__ float generic_row<4>(const uint8_t* r, const float* x, uint32_t K, int lane) {
    float acc = 0.f;
    for (uint32_t b = lane; b < K / 32; b += 32) {
        const uint8_t* q = r + (size_t)b * 20;
        float s = 0.f, xs = 0.f;
        for (int j = 0; j < 16; ++j) {
            const float x0 = x[b * 32 + j], x1 = x[b * 32 + 16 + j];
            s += (float)(q[4 + j] & 15) * x0 + (float)(q[4 + j] >> 4) * x1;
            xs += x0 + x1;
        }
        acc += s * ldh(q) + xs * ldh(q + 2);
    }
    return acc;
}
template <> __device__ float generic_row<5>(const uint8_t* r, const float* x, uint32_t K, int lane) {
    float acc = 0.f;
    // one (super-block, sub-block) pair per lane iteration
    for (uint32_t u = lane; u < K / 32; u += 32) {
        const uint8_t* q = r + (size_t)(u >> 3) * 176;
        const uint32_t j = u & 7, g = j >> 1, hi = j & 1;
        const uint8_t* sc = q + 4;
        uint32_t s6, m6;
        if (j < 4) { s6 = sc[j] & 63u; m6 = sc[j + 4] & 63u; }
        else { s6 = (sc[j + 4] & 15u) | ((sc[j - 4] >> 6) << 4); m6 = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
        float s = 0.f, xs = 0.f;
        for (int l = 0; l < 32; ++l) {
            const uint32_t nib = hi ? (q[48 + 32 * g + l] >> 4) : (q[48 + 32 * g + l] & 15u);
            const uint32_t code = nib + (((q[16 + l] >> j) & 1u) << 4);
            const float xv = x[(u >> 3) * 256 + j * 32 + l];
            s += (float)code * xv; xs += xv;
        }
        acc += ldh(q) * (float)s6 * s - ldh(q + 2) * (float)m6 * xs;
    }
    return acc;
}
template <> __device__ float generic_row<8>(const uint8_t* r, const float* x, uint32_t K, int lane) {
    float acc = 0.f;
    for (uint32_t u = lane; u < K / 32; u += 32) {          // one (super-block, sub-block) pair per lane iteration
        const uint8_t* q = r + (size_t)(u >> 3) * 144;
        const uint32_t j = u & 7, g = j >> 1, hi = j & 1;
        const uint8_t* sc = q + 4;
        uint32_t s6, m6;
        if (j < 4) { s6 = sc[j] & 63u; m6 = sc[j + 4] & 63u; }
        else { s6 = (sc[j + 4] & 15u) | ((sc[j - 4] >> 6) << 4); m6 = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
        float s = 0.f, xs = 0.f;
        for (int l = 0; l < 32; ++l) {
            const uint32_t code = hi ? (q[16 + 32 * g + l] >> 4) : (q[16 + 32 * g + l] & 15u);
            const float xv = x[(u >> 3) * 256 + j * 32 + l];
            s += (float)code * xv; xs += xv;
        }
        acc += ldh(q) * (float)s6 * s - ldh(q + 2) * (float)m6 * xs;
    }
    return acc;
}
template <> __device__ float generic_row<6>(const uint8_t* r, const float* x, uint32_t K, int lane) {
    float acc = 0.f;
    // one 16-weight sub-block per lane iteration: sub = 8h + 2j + (l/16)
    for (uint32_t u = lane; u < K / 16; u += 32) {
        const uint8_t* q = r + (size_t)(u >> 4) * 210;
        const uint32_t sub = u & 15, h = sub >> 3, j = (sub >> 1) & 3, l0 = (sub & 1) * 16;
        float s = 0.f;
        for (uint32_t l = l0; l < l0 + 16; ++l) {
            const uint8_t qlb = q[64 * h + 32 * (j & 1) + l];
            const uint32_t lo = (j & 2) ? (qlb >> 4) : (qlb & 15u);
            const uint32_t hi2 = (q[128 + 32 * h + l] >> (2 * j)) & 3u;
            s += (float)((int)(lo | (hi2 << 4)) - 32) * x[(u >> 4) * 256 + 128 * h + 32 * j + l];
        }
        acc += ldh(q + 208) * (float)(int8_t)q[192 + sub] * s;
    }
    return acc;
}

template <int DT>
__global__ void __launch_bounds__(256) gemv_generic(const GemvParams p) {
    extern __shared__ __align__(16) float xs[];            // transformed x, only when a fused transform is requested
    __shared__ float red[8];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    exchange_wait(p.xc, p.status);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* x = p.x;
    if (p.x_op != 0u) {
        float inv = 1.f;
        if (p.x_op == 1u) {
            float ss = 0.f;
            for (uint32_t i = threadIdx.x; i < p.K; i += blockDim.x) { const float t = p.x[i]; ss = fmaf(t, t, ss); }
#pragma unroll
            for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) red[warp] = ss;
            __syncthreads();
            float tot = 0.f;
            for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
            inv = 1.0f / sqrtf(tot / (float)p.K + p.eps);
        }
        for (uint32_t i = threadIdx.x; i < p.K; i += blockDim.x) {
            const float t = p.x[i];
            xs[i] = p.x_op == 1u ? t * inv * p.x2[i] : t / (1.0f + expf(-t)) * p.x2[i];
        }
        __syncthreads();
        x = xs;
    }
    const uint32_t cta_lo = blockIdx.x * (blockDim.x >> 5), row = cta_lo + warp;
    if (row < p.N) {
        float v = generic_row<DT>(row_ptr(p, row), x, p.K, lane);
#pragma unroll
        for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        const uint32_t e = y_index(p, row);
        if (lane == 0) store_row(p, e, p.accumulate ? p.y[e] + v : v);
    }
    exchange_signal(p.xc);
}

constexpr size_t kSmemLimit = 227 * 1024 - 256;          // dynamic part; the kernel also has a few static words
constexpr size_t kHalfSmem = 112 * 1024;                 // two such CTAs (of two kernels) fit one SM

// Bytes of shared memory outside the stage rings.
template <int DT> size_t stream_fixed_smem(unsigned K) {
    using L = Lane<DT>;
    const size_t nchunks = (K + L::STEP_W - 1) / L::STEP_W;
    return ((nchunks * 32 * L::XW * 4 + 127) / 128) * 128 + ((kMaxWarps * kMaxStages * 8 + 127) / 128) * 128 + 128;
}
unsigned g_last_grid = 0;
int env_int(const char* name, int dflt) {
    const char* e = std::getenv(name);
    return e && *e ? std::atoi(e) : dflt;
}

template <int DT, int R, int kWarps>
bool launch_stream_r(GemvParams p, unsigned stages, unsigned grid, size_t smem, unsigned cluster, cudaStream_t st) {
    p.stages = stages;
    static bool attr_set = false;
    static const bool pdl = env_int("TM_GEMV_PDL", 1) != 0;     // A/B knob: 0 launches without programmatic serialization
    if (!attr_set) {
        if (cudaFuncSetAttribute(gemv_stream<DT, R, kWarps>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit) != cudaSuccess)
            return fail("gemv: cannot raise the dynamic shared memory limit");
        // every GEMV asks for the largest shared-memory carveout, so consecutive kernels share one SM configuration
        cudaFuncSetAttribute(gemv_stream<DT, R, kWarps>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        attr_set = true;
    }
    if (cluster > 1) grid = (grid + cluster - 1) / cluster * cluster;      // CTAs past the last row only help stage x
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kWarps * 32); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[2];
    unsigned na = 0;
    if (pdl) {
        at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (cluster > 1) {
        at[na].id = cudaLaunchAttributeClusterDimension;
        at[na].val.clusterDim.x = cluster; at[na].val.clusterDim.y = 1; at[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = at; cfg.numAttrs = na;
    if (cudaLaunchKernelEx(&cfg, gemv_stream<DT, R, kWarps>, p) != cudaSuccess) return check_launch("gemv_stream");
    g_last_grid = grid;
    note_launch();
    return true;
}

// How many SMs a launch of one full-SM CTA per SM can cover when its CTAs come in clusters of `cluster`
// (clusters live inside one GPC, so a GPC whose SM count is not a multiple of the cluster size leaves
// SMs unused). Asked of the driver once per cluster size.
template <int DT, int kWarps>
unsigned cluster_sms(unsigned cluster, unsigned sms) {
    static unsigned cached[9] = {};
    if (cluster <= 1 || cluster > 8) return sms;
    if (!cached[cluster]) {
        cudaFuncSetAttribute(gemv_stream<DT, 1, kWarps>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(sms / cluster * cluster); cfg.blockDim = dim3(kWarps * 32);
        cfg.dynamicSmemBytes = kWarps == 16 ? kSmemLimit : kHalfSmem;       // one CTA per SM (16 warps) or two (8 warps)
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = cluster; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemv_stream<DT, 1, kWarps>, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = 0; }
        unsigned got = (unsigned)n * cluster;
        if (kWarps == 8) got /= 2;                                          // counted two CTAs per SM
        cached[cluster] = got > sms ? sms : (got ? got : 1u);               // 1: clusters of this size do not fit at all
    }
    return cached[cluster];
}

template <int DT> bool launch_generic_only(GemvParams p, cudaStream_t st);

template <int DT>
bool launch_dt(GemvParams p, bool aligned, cudaStream_t st) {
    using L = Lane<DT>;
    const unsigned nchunks = (p.K + L::STEP_W - 1) / L::STEP_W;
    if (aligned && nchunks <= (unsigned)kMaxWarps) {
        const unsigned sms = (unsigned)device_sm_count();
        static const int force_r = env_int("TM_GEMV_R", 0), force_s = env_int("TM_GEMV_STAGES", 0),
                         force_w = env_int("TM_GEMV_WARPS", 0);
        // One 16-warp CTA per SM. 8-warp CTAs (TM_GEMV_WARPS=8) were the rule for matrices with fewer than 8 rows
        // per SM until the x staging was reworked; they now cost 4 % on the ten-GEMV sweep (70.5 vs 68.0 us).
        // TM_GEMV_HALF_MB > 0 (an experiment, off by default) gives matrices up to that many MB an 8-warp
        // CTA limited to half of an SM's shared memory, so that two consecutive kernels can be resident
        // together; measured slower (sweep 78 vs 65 us, 8B chain 3.2 vs 2.7 ms per token): 8 warps do not
        // decode fast enough.
        static const int half_mb = env_int("TM_GEMV_HALF_MB", 0);
        const bool half = half_mb > 0 && nchunks <= 8 && (size_t)p.N * p.row_bytes <= (size_t)half_mb << 20;
        int warps_cta = half ? 8 : 16;
        if ((force_w == 8 && nchunks <= 8) || force_w == 16) warps_cta = force_w;
        const size_t smem_limit = half ? kHalfSmem : kSmemLimit;
        // Clusters can share the staging of x (see the kernel). Off by default: measured on B200, launching the
        // GEMVs as clusters of 2 or 4 made every launch slower by more than the staging it saved (ten-GEMV
        // sweep 129 vs 72 us, 8B chain 2.9 vs 2.25 ms per token; staging of K = 14336 fell from 10 to 5.7 us
        // but the time from staged x to the last row grew by 6 us). TM_GEMV_CLUSTER=2 or 4 turns them on.
        static const int force_c = env_int("TM_GEMV_CLUSTER", 1);
        unsigned cluster = 1u;
        if ((force_c == 2 || force_c == 4) && !p.xq) cluster = (unsigned)force_c;
        unsigned sms_c = sms;
        while (cluster > 1) {
            sms_c = warps_cta == 16 ? cluster_sms<DT, 16>(cluster, sms) : cluster_sms<DT, 8>(cluster, sms);
            if (sms_c * 16 >= sms * 15) break;               // at most 1/16 of the SMs lost to the cluster shape
            cluster >>= 1; sms_c = sms;
        }
        const unsigned teams = (unsigned)warps_cta / nchunks;
        unsigned grid = (p.N + teams - 1) / teams;
        if (grid > sms_c) grid = sms_c;
        p.rows_per_cta = (p.N + grid - 1) / grid;
        grid = (p.N + p.rows_per_cta - 1) / p.rows_per_cta;
        const unsigned rows_per_team = (p.rows_per_cta + teams - 1) / teams;
        // Rows per ring item: as many as a team's share offers (the step's activations stay in
        // registers across them), at most 4, and few enough that at least two stages fit.
        int R = rows_per_team >= 4 ? 4 : rows_per_team >= 2 ? 2 : 1;
        if (force_r == 1 || force_r == 2 || force_r == 4) R = force_r;
        const size_t fixed = stream_fixed_smem<DT>(p.K) + (nchunks > 1 ? (size_t)p.rows_per_cta * nchunks * 4 : 0);
        auto fit = [&](int r) -> unsigned {
            const size_t per = (size_t)warps_cta * r * L::STEP_BYTES;
            if (fixed + 2 * per > smem_limit) return 0u;
            const size_t s = (smem_limit - fixed) / per;
            return (unsigned)(s > (size_t)kMaxStages ? kMaxStages : s);
        };
        while (R > 1 && fit(R) < 2) R >>= 1;
        unsigned S = fit(R);
        if (S >= 2) {
            // No deeper than a warp has items, and by default no deeper than 3: the ring only has
            // to cover the DRAM latency.
            const unsigned items = (rows_per_team + R - 1) / R;
            // The half-SM shape prefetches while the previous kernel runs: as deep as the warp has items.
            unsigned cap = force_s >= 2 ? (unsigned)force_s : (half ? (unsigned)kMaxStages : 3u);
            if (cap > (unsigned)kMaxStages) cap = kMaxStages;
            if (S > cap) S = cap;
            if (S > items) S = items < 1 ? 1 : items;
            const size_t smem = fixed + (size_t)S * warps_cta * R * L::STEP_BYTES;
            if (warps_cta == 16) {
                switch (R) {
                    case 4: return launch_stream_r<DT, 4, 16>(p, S, grid, smem, cluster, st);
                    case 2: return launch_stream_r<DT, 2, 16>(p, S, grid, smem, cluster, st);
                    default: return launch_stream_r<DT, 1, 16>(p, S, grid, smem, cluster, st);
                }
            }
            switch (R) {
                case 4: return launch_stream_r<DT, 4, 8>(p, S, grid, smem, cluster, st);
                case 2: return launch_stream_r<DT, 2, 8>(p, S, grid, smem, cluster, st);
                default: return launch_stream_r<DT, 1, 8>(p, S, grid, smem, cluster, st);
            }
        }
    }
    return launch_generic_only<DT>(p, st);
}

template <int DT>
bool launch_generic_only(GemvParams p, cudaStream_t st) {
    p.xq = nullptr;                                         // the plain kernel reads the fp32 x
    const unsigned rows_per_cta = 8;
    const size_t xsmem = p.x_op ? (size_t)p.K * 4 : 0;
    if (xsmem > 48 * 1024) {
        static bool attr = false;
        if (!attr && cudaFuncSetAttribute(gemv_generic<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
            return fail("gemv: cannot raise the dynamic shared memory limit");
        attr = true;
        if (xsmem > 200 * 1024) return fail("gemv: K=%u is too long for the unaligned fused form", p.K);
    }
    gemv_generic<DT><<<(p.N + rows_per_cta - 1) / rows_per_cta, rows_per_cta * 32, xsmem, st>>>(p);
    g_last_grid = (p.N + rows_per_cta - 1) / rows_per_cta;
    note_launch();
    return check_launch("gemv_generic");
}

bool launch_any(const GemvParams& p, unsigned dtype, bool aligned, cudaStream_t st) {
    switch (dtype) {
        case DT_Q8_0: return launch_dt<0>(p, aligned, st);
        case DT_Q4_0: return launch_dt<1>(p, aligned, st);
        case DT_Q4_1: return launch_dt<4>(p, aligned, st);
        case DT_Q5_K: return launch_dt<5>(p, aligned, st);
        case DT_Q4_K: return launch_dt<8>(p, aligned, st);
        case DT_GGUF_Q4_0: return launch_dt<9>(p, aligned, st);
        default: return launch_dt<6>(p, aligned, st);
    }
}
}  // namespace

unsigned last_gemv_grid() { return g_last_grid; }

bool launch_gemv(const float* x, const uint8_t* W, float* y, unsigned N, unsigned K, unsigned dtype,
                 const SegTable& seg, cudaStream_t st, const GemvFuse* fuse) {
    const unsigned be = block_elems(dtype);
    if (!be || dtype == DT_F16) return fail("gemv: dtype %u is not a block format", dtype);
    if (!x || !W || !y) return fail("gemv: null pointer");
    if (N == 0) return true;
    if (K == 0 || K % be) return fail("gemv: K=%u is not a multiple of %u", K, be);
    if (seg.nseg == 0 || seg.nseg > (unsigned)kMaxSeg) return fail("gemv: %u segments (1..%d supported)", seg.nseg, kMaxSeg);
    if (seg.row_end[seg.nseg - 1] != N) return fail("gemv: segment rows do not add up to N");
    if ((uintptr_t)x % 16) return fail("gemv: x must be 16-byte aligned");
    GemvParams p;
    p.W = W; p.x = x; p.y = y; p.N = N; p.K = K;
    p.row_bytes = (K / be) * block_bytes(dtype);
    p.seg = seg; p.status = device_status_word(); p.trace = device_trace();
    p.x2 = nullptr; p.eps = 0.f; p.x_op = 0; p.accumulate = 0;
    p.xc = Exchange{};
    p.xq = nullptr;
    if (fuse && fuse->xchg) p.xc = *fuse->xchg;
    if (p.xc.npush > (unsigned)kMaxPeers || (p.xc.nwait && (!p.xc.wait_ctrs || !p.xc.wait_ctas || !p.xc.epoch)))
        return fail("gemv: incomplete peer exchange description");
    if (fuse) {
        if (fuse->x_op > 2 || (fuse->x_op != 0 && (!fuse->x2 || (uintptr_t)fuse->x2 % 16))) return fail("gemv: bad fused x transform");
        p.x2 = fuse->x2; p.eps = fuse->eps; p.x_op = fuse->x_op; p.accumulate = fuse->accumulate ? 1u : 0u;
        if (fuse->xq) {
            if ((uintptr_t)fuse->xq % 16) return fail("gemv: the staged x image must be 16-byte aligned");
            p.xq = fuse->xq;
        }
    }
    bool aligned = ((uintptr_t)W % 16 == 0) && (p.row_bytes % 16 == 0);
    for (unsigned s = 0; s < seg.nseg; ++s) aligned = aligned && (seg.woff[s] % 16 == 0);
    if (dtype == DT_TQ2) {                                  // ternary rows: the plain kernel (no streaming lane is built for them)
        p.xq = nullptr;
        return launch_generic_only<7>(p, st);
    }
    return launch_any(p, dtype, aligned, st);
}

size_t xq_bytes(unsigned K, unsigned dtype) {
    auto sz = [&](unsigned step_w, unsigned xw) { return (size_t)kXqHeaderWords * 4 + (size_t)((K + step_w - 1) / step_w) * 32u * xw * 4u; };
    switch (dtype) {
        case DT_Q8_0: return sz(Lane<0>::STEP_W, Lane<0>::XW);
        case DT_Q4_0: return sz(Lane<1>::STEP_W, Lane<1>::XW);
        case DT_Q4_1: return sz(Lane<4>::STEP_W, Lane<4>::XW);
        case DT_Q5_K: return sz(Lane<5>::STEP_W, Lane<5>::XW);
        case DT_Q4_K: return sz(Lane<8>::STEP_W, Lane<8>::XW);
        case DT_GGUF_Q4_0: return sz(Lane<9>::STEP_W, Lane<9>::XW);
        case DT_Q6_K: return sz(Lane<6>::STEP_W, Lane<6>::XW);
        default: return 0;
    }
}

namespace {
template <int CDT>
bool launch_xprep_dt(uint32_t* out, const float* x, const float* x2, unsigned x_op, float eps, unsigned K, const Exchange& xc, cudaStream_t st) {
    const unsigned ngroups = (K + 255u) / 256u;
    // RMSNorm sums over the whole vector: one CTA of 16 warps. Otherwise four groups per CTA.
    const unsigned threads = x_op == 1u ? 512u : 128u, grid = x_op == 1u ? 1u : (ngroups + 3u) / 4u;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(threads); cfg.dynamicSmemBytes = 0; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, xprep_kernel<CDT>, out, x, x2, (uint32_t)x_op, eps, (uint32_t)K, xc, device_status_word()) != cudaSuccess)
        return check_launch("xprep");
    note_launch();
    return true;
}
}  // namespace

bool launch_xprep(uint32_t* out, const float* x, const float* x2, unsigned x_op, float eps, unsigned K, unsigned dtype,
                  const Exchange* xchg, cudaStream_t st) {
    if (!out || !x || (uintptr_t)out % 16 || (uintptr_t)x % 16 || x_op > 2 || (x_op && (!x2 || (uintptr_t)x2 % 16)))
        return fail("xprep: bad arguments");
    const unsigned be = block_elems(dtype);
    if (!be || dtype == DT_F16 || K == 0 || K % be) return fail("xprep: K=%u is not whole blocks of dtype %u", K, dtype);
    const Exchange xc = xchg ? *xchg : Exchange{};
    switch (dtype) {
        case DT_Q8_0: return launch_xprep_dt<0>(out, x, x2, x_op, eps, K, xc, st);
        case DT_Q4_0: return launch_xprep_dt<1>(out, x, x2, x_op, eps, K, xc, st);
        case DT_Q4_1: return launch_xprep_dt<4>(out, x, x2, x_op, eps, K, xc, st);
        case DT_Q5_K: return launch_xprep_dt<5>(out, x, x2, x_op, eps, K, xc, st);
        case DT_Q4_K: return launch_xprep_dt<8>(out, x, x2, x_op, eps, K, xc, st);
        case DT_GGUF_Q4_0: return launch_xprep_dt<9>(out, x, x2, x_op, eps, K, xc, st);
        default: return launch_xprep_dt<6>(out, x, x2, x_op, eps, K, xc, st);
    }
}

}  // namespace tmc
