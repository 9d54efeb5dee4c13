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
//   * x is staged once per CTA into swizzled shared memory together with its
//     per-32-block sums (used to strip code offsets and zero points).
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

namespace tmc {

namespace {

constexpr int kWarps = 8;          // warps per CTA
constexpr int kMaxStages = 8;      // ring depth per warp is chosen at launch, 2..kMaxStages
constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // a copy that has not landed in 2 s never will

struct GemvParams {
    const uint8_t* W;
    const float* x;
    float* y;
    uint32_t N, K, row_bytes;
    uint32_t stages;
    SegTable seg;
    int* status;
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
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: false when the time limit ran out (the caller records it and leaves).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned long long limit_ns = kWaitLimitNs) {
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

__device__ __forceinline__ const uint8_t* row_ptr(const GemvParams& p, uint32_t row) {
    uint32_t s = 0, start = 0;
    while (s + 1 < p.seg.nseg && row >= p.seg.row_end[s]) { start = p.seg.row_end[s]; ++s; }
    return p.W + p.seg.woff[s] + (size_t)(row - start) * p.row_bytes;
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

// Shared memory: [x: padded K floats, swizzled float4 slots][xsum: padded K/32][mbarriers][stages]
template <int DT, int R>
__global__ void __launch_bounds__(kWarps * 32, 1) gemv_stream(const GemvParams p) {
    using L = Lane<DT>;
    constexpr int ROWCAP = L::STEP_BYTES;                  // multiple of 16
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t nchunks = (p.K + L::STEP_W - 1) / L::STEP_W;
    const uint32_t kpad = nchunks * L::STEP_W;
    float4* xs4 = reinterpret_cast<float4*>(smem);
    float* xsum = reinterpret_cast<float*>(smem + (size_t)kpad * 4);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kpad * 4 + (size_t)(kpad / 32) * 4);
    const uint32_t S = p.stages;
    uint8_t* stages = reinterpret_cast<uint8_t*>(bars) + ((kWarps * kMaxStages * 8 + 127) / 128) * 128;
    uint64_t* mybar = bars + warp * kMaxStages;
    uint8_t* mystage = stages + (size_t)warp * S * R * ROWCAP;

    const uint32_t ngroups = (p.N + R - 1) / R;
    const uint32_t gwarp = blockIdx.x * kWarps + warp, nwarps = gridDim.x * kWarps;
    const uint32_t mygroups = ngroups > gwarp ? (ngroups - gwarp + nwarps - 1) / nwarps : 0;
    const uint32_t items = mygroups * nchunks;

    if (lane == 0) {
        for (uint32_t s = 0; s < S; ++s) mbar_init(&mybar[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    // item t -> (row group, chunk); lane 0 posts the R row copies of the item into ring slot `slot`
    auto issue = [&](uint32_t t, uint32_t slot) {
        const uint32_t g = gwarp + (t / nchunks) * nwarps, c = t % nchunks;
        const uint32_t off = c * (uint32_t)L::STEP_BYTES;
        const uint32_t bytes = min((uint32_t)L::STEP_BYTES, p.row_bytes - off);
        uint64_t* bar = &mybar[slot];
        uint8_t* dst = mystage + (size_t)slot * R * ROWCAP;
        uint32_t rows = min((uint32_t)R, p.N - g * R);
        mbar_expect_tx(bar, rows * bytes);
        for (uint32_t r = 0; r < rows; ++r)
            bulk_g2s(dst + r * ROWCAP, row_ptr(p, g * R + r) + off, bytes, bar);
    };
    if (lane == 0)
        for (uint32_t t = 0; t < items && t < S; ++t) issue(t, t);

    // Everything above touches only weights. x may be written by the preceding
    // kernel in the stream: wait for it here, and let the next kernel start its own
    // weight prefetch.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // ---- stage x (swizzled) and its 32-block sums --------------------------
    const float4* xg4 = reinterpret_cast<const float4*>(p.x);
    for (uint32_t q = threadIdx.x; q < kpad / 4; q += blockDim.x) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (q * 4 < p.K) v = __ldcg(xg4 + q);                // K is a multiple of 32
        xs4[x_slot(q)] = v;
    }
    for (uint32_t b = threadIdx.x; b < kpad / 32; b += blockDim.x) {
        float s = 0.f;
        if (b * 32 < p.K) {
#pragma unroll
            for (int i = 0; i < 8; ++i) { const float4 v = __ldcg(xg4 + b * 8 + i); s += (v.x + v.y) + (v.z + v.w); }
        }
        xsum[b] = s;
    }
    __syncthreads();

    // ---- consume -------------------------------------------------------------
    typename L::X xr;
    float acc[R];
    bool dead = false;
    uint32_t slot = 0, phase = 0, k = 0, c = 0;
    for (uint32_t t = 0; t < items; ++t) {
        if (c == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r] = 0.f;
        }
        if (nchunks > 1 || t == 0) L::load_x(xr, xs4, xsum, (int)c, lane);
        if (!mbar_wait(&mybar[slot], phase)) { dead = true; break; }
        const uint32_t wchunk = min((uint32_t)L::STEP_W, p.K - c * L::STEP_W);
        const int valid = lane_valid<DT>(lane, (int)(wchunk / L::UNIT_W));
        const uint8_t* st = mystage + (size_t)slot * R * ROWCAP;
        if (L::LANE_UNITS == 2 ? valid > 0 : true) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint8_t* rowp = st + r * ROWCAP + (L::LANE_UNITS == 2 ? lane * L::LANE_BYTES : 0);
                acc[r] += L::dot(rowp, xr, lane, valid);
            }
        }
        __syncwarp();                                       // every lane is done with this stage
        if (lane == 0 && t + S < items) issue(t + S, slot);
        if (++slot == S) { slot = 0; phase ^= 1u; }
        if (c + 1 == nchunks) {
            const uint32_t row0 = (gwarp + k * nwarps) * R;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float v = acc[r];
#pragma unroll
                for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == r && row0 + r < p.N) p.y[row0 + r] = v;
            }
            c = 0; ++k;
        } else {
            ++c;
        }
    }
    if (dead) {
        // A copy never completed. Record it, give the copies still in flight a last
        // bounded chance to land (they target this CTA's shared memory) and leave.
        if (lane == 0) {
            atomicExch(p.status, 1);
            for (uint32_t s = 0; s < S; ++s) (void)mbar_wait(&mybar[s], 0, 50000000ull), (void)mbar_wait(&mybar[s], 1, 50000000ull);
        }
    }
}

// Rows beyond N inside a group are never copied; their lanes multiply stale stage
// bytes and the result is dropped at the store, so nothing there needs clearing.

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
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= p.N) return;
    float v = generic_row<DT>(row_ptr(p, row), p.x, p.K, lane);
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) p.y[row] = v;
}

constexpr size_t kSmemLimit = 227 * 1024;

// Bytes of shared memory outside the stage rings.
template <int DT> size_t stream_fixed_smem(unsigned K) {
    using L = Lane<DT>;
    const size_t nchunks = (K + L::STEP_W - 1) / L::STEP_W, kpad = nchunks * L::STEP_W;
    return kpad * 4 + kpad / 32 * 4 + ((kWarps * kMaxStages * 8 + 127) / 128) * 128 + 128;
}
// Deepest ring (<= kMaxStages) that fits next to x; 0 when not even two stages fit.
template <int DT> unsigned stream_stages(unsigned K, int R) {
    using L = Lane<DT>;
    const size_t fixed = stream_fixed_smem<DT>(K), per = (size_t)kWarps * R * L::STEP_BYTES;
    if (fixed + 2 * per > kSmemLimit) return 0;
    const size_t s = (kSmemLimit - fixed) / per;
    return (unsigned)(s > (size_t)kMaxStages ? kMaxStages : s);
}

template <int DT, int R>
bool launch_stream_r(GemvParams p, cudaStream_t st) {
    using L = Lane<DT>;
    p.stages = stream_stages<DT>(p.K, R);
    const size_t smem = stream_fixed_smem<DT>(p.K) + (size_t)p.stages * kWarps * R * L::STEP_BYTES;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(gemv_stream<DT, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit) != cudaSuccess)
            return fail("gemv: cannot raise the dynamic shared memory limit");
        attr_set = true;
    }
    const unsigned ngroups = (p.N + R - 1) / R;
    unsigned grid = (ngroups + kWarps - 1) / kWarps;
    const unsigned sms = (unsigned)device_sm_count();
    if (grid > sms) grid = sms;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kWarps * 32); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, gemv_stream<DT, R>, p) != cudaSuccess) return check_launch("gemv_stream");
    note_launch();
    return true;
}

template <int DT>
bool launch_dt(const GemvParams& p, bool aligned, cudaStream_t st) {
    using L = Lane<DT>;
    if (aligned) {
        // Rows per warp task: 4 when that still gives every warp of the machine a
        // task, fewer for short matrices so the rows spread over more SMs.
        const unsigned warps = (unsigned)device_sm_count() * kWarps;
        int R = 4;
        if ((p.N + 3) / 4 < warps) R = 2;
        if ((p.N + 1) / 2 < warps) R = 1;
        while (R > 1 && stream_stages<DT>(p.K, R) < 3) R >>= 1;
        if (stream_stages<DT>(p.K, R) >= 2) {
            switch (R) {
                case 4: return launch_stream_r<DT, 4>(p, st);
                case 2: return launch_stream_r<DT, 2>(p, st);
                default: return launch_stream_r<DT, 1>(p, st);
            }
        }
    }
    (void)sizeof(L);
    const unsigned rows_per_cta = 8;
    gemv_generic<DT><<<(p.N + rows_per_cta - 1) / rows_per_cta, rows_per_cta * 32, 0, st>>>(p);
    note_launch();
    return check_launch("gemv_generic");
}

}  // namespace

bool launch_gemv(const float* x, const uint8_t* W, float* y, unsigned N, unsigned K, unsigned dtype,
                 const SegTable& seg, cudaStream_t st) {
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
    p.seg = seg; p.status = device_status_word();
    bool aligned = ((uintptr_t)W % 16 == 0) && (p.row_bytes % 16 == 0);
    for (unsigned s = 0; s < seg.nseg; ++s) aligned = aligned && (seg.woff[s] % 16 == 0);
    switch (dtype) {
        case DT_Q8_0: return launch_dt<0>(p, aligned, st);
        case DT_Q4_0: return launch_dt<1>(p, aligned, st);
        case DT_Q4_1: return launch_dt<4>(p, aligned, st);
        case DT_Q5_K: return launch_dt<5>(p, aligned, st);
        default: return launch_dt<6>(p, aligned, st);
    }
}

}  // namespace tmc
