// attn_fused.cu — one-launch decode attention of the chain lane: rope(q), rope(k) -> K cache,
// v -> V cache, GQA split-K attention and the merge of the splits.
//
// The reference runs this as five dispatches (tensormark/metal.h:3950-3967 rope_q, 3968-4005
// rope_k_cache, 4006-4030 v_cache, 2739-2859 / 4153-4222 attention and its split merge). On a GPU
// whose GEMVs take a few microseconds each, five launches with a dependent chain of cache misses
// behind each cost more than the attention itself, so the chain form does it in one kernel:
//
//   grid (KVH, nsplit), 4 warps. The positions [0, pos] are cut into tiles of 32; a CTA owns a
//   contiguous range of tiles of one KV head and its warps take them round-robin.
//   * Every CTA rotates the REP query heads of its KV head into shared memory (q is tiny).
//   * The CTA whose range holds position `pos` rotates the new k, stores k and v into the caches
//     and, after a barrier, reads them back like any other position.
//   * Scores: one LANE per POSITION. A lane reads its own K row (contiguous) and dots it with the
//     query heads from shared memory (broadcast reads): no shuffle per position, 32 independent
//     row reads in flight per warp.
//   * Values: one lane per dh/32 DIMS. For each position of the tile the lanes read one V row
//     (coalesced) and the position's weights come by shuffle.
//   * A CTA leaves an unnormalised partial (max, sum, acc) per head; the CTA that arrives last at a
//     KV head's counter merges the nsplit partials and writes the output rows.
//
// The arithmetic is the reference's (fp32 scores, exp of score - max, value sum, one division);
// only the order of the sums differs, so results agree with the oracle to rounding.
#include "common.cuh"
#include "glue.h"

#include <cstdlib>

#include <cuda_fp16.h>
#include <math_constants.h>

namespace tmc {

namespace {

constexpr unsigned kMaxSplits = 32;      // merge scratch in shared memory: 2 * REP * kMaxSplits floats

__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename T> __device__ __forceinline__ T to_cache(float v);
template <> __device__ __forceinline__ float to_cache<float>(float v) { return v; }
template <> __device__ __forceinline__ __half to_cache<__half>(float v) { return __float2half_rn(v); }

// Raw loads are issued in batches before anything is computed on them: the kernel is a chain of
// cache-miss latencies, so what matters is how many loads are in flight, not how many are issued.
template <typename T> struct Raw8;
template <> struct Raw8<__half> { uint4 u; };
template <> struct Raw8<float> { float4 a, b; };
__device__ __forceinline__ void fetch8(const __half* p, Raw8<__half>& r) { r.u = __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void fetch8(const float* p, Raw8<float>& r) {
    r.a = __ldcg(reinterpret_cast<const float4*>(p)); r.b = __ldcg(reinterpret_cast<const float4*>(p) + 1);
}
__device__ __forceinline__ void unpack8(const Raw8<__half>& r, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&r.u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ void unpack8(const Raw8<float>& r, float (&f)[8]) {
    f[0] = r.a.x; f[1] = r.a.y; f[2] = r.a.z; f[3] = r.a.w; f[4] = r.b.x; f[5] = r.b.y; f[6] = r.b.z; f[7] = r.b.w;
}
// DPL consecutive cache elements (DPL = 2 or 4): raw fetch now, floats later.
template <typename T, int DPL> struct RawV;
template <> struct RawV<__half, 4> { uint2 u; };
template <> struct RawV<__half, 2> { unsigned u; };
template <> struct RawV<float, 4> { float4 u; };
template <> struct RawV<float, 2> { float2 u; };
__device__ __forceinline__ void fetchv(const __half* p, RawV<__half, 4>& r) { r.u = __ldcg(reinterpret_cast<const uint2*>(p)); }
__device__ __forceinline__ void fetchv(const __half* p, RawV<__half, 2>& r) { r.u = __ldcg(reinterpret_cast<const unsigned*>(p)); }
__device__ __forceinline__ void fetchv(const float* p, RawV<float, 4>& r) { r.u = __ldcg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ void fetchv(const float* p, RawV<float, 2>& r) { r.u = __ldcg(reinterpret_cast<const float2*>(p)); }
__device__ __forceinline__ void unpackv(const RawV<__half, 4>& r, float (&f)[4]) {
    const __half2* h = reinterpret_cast<const __half2*>(&r.u);
    const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ void unpackv(const RawV<__half, 2>& r, float (&f)[2]) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r.u));
    f[0] = a.x; f[1] = a.y;
}
__device__ __forceinline__ void unpackv(const RawV<float, 4>& r, float (&f)[4]) { f[0] = r.u.x; f[1] = r.u.y; f[2] = r.u.z; f[3] = r.u.w; }
__device__ __forceinline__ void unpackv(const RawV<float, 2>& r, float (&f)[2]) { f[0] = r.u.x; f[1] = r.u.y; }

template <typename T, int DPL, int REP>
__global__ void __launch_bounds__(128) attn_fused_kernel(const float* qkv, T* kc, T* vc, float* part, float* stat,
                                                          unsigned* counters, float* out, uint32_t H, uint32_t KVH,
                                                          uint32_t ctx, float scale, const float2* __restrict__ tbl,
                                                          uint32_t tbl_n, const int* st, unsigned long long* trace) {
    unsigned long long* tr = nullptr;                         // timeline of CTA (0, 0), thread 0 (see tm_cuda_trace_read)
    if (trace && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) {
        const unsigned long long slot = atomicAdd(trace, 1ull);
        if (slot < (unsigned long long)kTraceLaunches) { tr = trace + 1 + slot * kTraceWords; tr[0] = now_ns(); }
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int dh = DPL * 32, half = dh / 2;
    const uint32_t kv = blockIdx.x, split = blockIdx.y, nsplit = gridDim.y;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // The position was written by the previous token's last kernel and the cache rows below it by earlier tokens:
    // both are safe to read before this token's q|k|v GEMV has finished, and this CTA is resident (and idle) for
    // several microseconds before that. So the first tile's loads, with their page walks and DRAM latency, are
    // requested now; only the row of the new position is fetched after it has been written.
    const int pos_i = *(volatile const int*)st;
    const bool valid = !(pos_i < 0 || (uint32_t)pos_i >= ctx || (uint32_t)pos_i * half + half > tbl_n);   // same guard as the separate kernels
    const uint32_t pos = valid ? (uint32_t)pos_i : 0u, allow = pos + 1;
    const uint32_t tiles = (allow + 31) / 32, tps = (tiles + nsplit - 1) / nsplit;
    const uint32_t t0 = min(tiles, split * tps), t1 = min(tiles, t0 + tps);
    const T* kbase = kc + (size_t)kv * ctx * dh;
    const T* vbase = vc + (size_t)kv * ctx * dh;
    Raw8<T> raw[dh / 8];
    RawV<T, DPL> vraw[32];                                     // rows past the tile's last position repeat it, their weight is 0
    auto fetch_tile = [&](uint32_t t) {                        // this lane's K row (lane = position) and its dims of the 32 V rows
        const uint32_t p = t * 32 + lane, np = min(32u, allow - t * 32);
        const T* krow = kbase + (size_t)min(p, allow - 1) * dh;
        const T* vrow = vbase + (size_t)t * 32 * dh + lane * DPL;
#pragma unroll
        for (int c = 0; c < dh / 8; ++c) fetch8(krow + c * 8, raw[c]);
#pragma unroll
        for (int k = 0; k < 32; ++k) fetchv(vrow + (size_t)min((uint32_t)k, np - 1) * dh, vraw[k]);
    };
    const uint32_t t_first = t0 + warp;
    if (valid && t_first < t1) fetch_tile(t_first);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tr) tr[1] = now_ns();
    if (!valid) return;

    __shared__ __align__(16) float qs[REP][dh];
    __shared__ float sm_acc[4][REP][dh];
    __shared__ float sm_m[4][REP], sm_l[4][REP];
    __shared__ int sm_last;

    // ---- rope(q) for this KV head's query heads, scaled, into shared memory
    for (uint32_t i = threadIdx.x; i < REP * half; i += 128) {
        const uint32_t r = i / half, j = i % half;
        const float2 cs = tbl[(size_t)pos * half + j];
        const float* q = qkv + (size_t)(kv * REP + r) * dh;
        const float a = __ldcg(q + j), b = __ldcg(q + j + half);
        qs[r][j] = (a * cs.x - b * cs.y) * scale;
        qs[r][j + half] = (b * cs.x + a * cs.y) * scale;
    }
    // ---- the new position's k (rotated) and v go into the caches; the CTA that attends it writes them
    if (t1 == tiles && t1 > t0) {
        const float* kn = qkv + (size_t)(H + kv) * dh;
        const float* vn = qkv + (size_t)(H + KVH + kv) * dh;
        T* kdst = kc + ((size_t)kv * ctx + pos) * dh;
        T* vdst = vc + ((size_t)kv * ctx + pos) * dh;
        for (uint32_t j = threadIdx.x; j < (uint32_t)half; j += 128) {
            const float2 cs = tbl[(size_t)pos * half + j];
            const float a = __ldcg(kn + j), b = __ldcg(kn + j + half);
            kdst[j] = to_cache<T>(a * cs.x - b * cs.y);
            kdst[j + half] = to_cache<T>(b * cs.x + a * cs.y);
        }
        for (uint32_t j = threadIdx.x; j < (uint32_t)dh; j += 128) vdst[j] = to_cache<T>(__ldcg(vn + j));
    }
    __syncthreads();
    if (tr) tr[2] = now_ns();

    // ---- this warp's tiles
    float m[REP], l[REP], acc[REP][DPL];
#pragma unroll
    for (int r = 0; r < REP; ++r) {
        m[r] = -CUDART_INF_F; l[r] = 0.f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[r][d] = 0.f;
    }
    for (uint32_t t = t_first; t < t1; t += 4) {
        const uint32_t p = t * 32 + lane;
        const bool live = p < allow;
        float s[REP];
#pragma unroll
        for (int r = 0; r < REP; ++r) s[r] = 0.f;
        // Every load of a tile is requested before anything is computed on it. The first tile's were requested
        // before the wait; of those, whatever aliases the new position's row is fetched again now that it is written.
        if (t != t_first) {
            fetch_tile(t);
        } else if (t == tiles - 1) {
            const uint32_t kpos = pos - t * 32;
            if (lane >= kpos) {
#pragma unroll
                for (int c = 0; c < dh / 8; ++c) fetch8(kbase + (size_t)pos * dh + c * 8, raw[c]);
            }
#pragma unroll
            for (int k = 0; k < 32; ++k)
                if ((uint32_t)k >= kpos) fetchv(vbase + (size_t)pos * dh + lane * DPL, vraw[k]);
        }
        if (live) {
#pragma unroll
            for (int c = 0; c < dh / 8; ++c) {
                float kf[8];
                unpack8(raw[c], kf);
#pragma unroll
                for (int r = 0; r < REP; ++r) {
                    const float4 qa = *reinterpret_cast<const float4*>(&qs[r][c * 8]);
                    const float4 qb = *reinterpret_cast<const float4*>(&qs[r][c * 8 + 4]);
                    float v = s[r];
                    v = fmaf(qa.x, kf[0], v); v = fmaf(qa.y, kf[1], v); v = fmaf(qa.z, kf[2], v); v = fmaf(qa.w, kf[3], v);
                    v = fmaf(qb.x, kf[4], v); v = fmaf(qb.y, kf[5], v); v = fmaf(qb.z, kf[6], v); v = fmaf(qb.w, kf[7], v);
                    s[r] = v;
                }
            }
        }
        // tile softmax statistics and this lane's weight per head
        float pw[REP];
#pragma unroll
        for (int r = 0; r < REP; ++r) {
            float tm = live ? s[r] : -CUDART_INF_F;
#pragma unroll
            for (int o = 16; o; o >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, o));
            const float mn = fmaxf(m[r], tm);                 // finite: every tile holds at least one live position
            const float corr = __expf(m[r] - mn);
            pw[r] = live ? __expf(s[r] - mn) : 0.f;
            float ts = pw[r];
#pragma unroll
            for (int o = 16; o; o >>= 1) ts += __shfl_xor_sync(0xffffffffu, ts, o);
            l[r] = l[r] * corr + ts;
#pragma unroll
            for (int d = 0; d < DPL; ++d) acc[r][d] *= corr;
            m[r] = mn;
        }
        // values: lanes own dims, the tile's positions one after another (weight 0 past the last position)
#pragma unroll
        for (int k = 0; k < 32; ++k) {
            float vf[DPL];
            unpackv(vraw[k], vf);
#pragma unroll
            for (int r = 0; r < REP; ++r) {
                const float w = __shfl_sync(0xffffffffu, pw[r], k);
#pragma unroll
                for (int d = 0; d < DPL; ++d) acc[r][d] = fmaf(w, vf[d], acc[r][d]);
            }
        }
    }

    if (tr) tr[4] = now_ns();
    // ---- merge the four warps, leave this split's partial
#pragma unroll
    for (int r = 0; r < REP; ++r) {
        if (lane == 0) { sm_m[warp][r] = m[r]; sm_l[warp][r] = l[r]; }
#pragma unroll
        for (int d = 0; d < DPL; ++d) sm_acc[warp][r][lane * DPL + d] = acc[r][d];
    }
    __syncthreads();
    for (int r = 0; r < REP; ++r) {
        float M = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w][r]);
        float Lsum = 0.f, f[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) { f[w] = sm_m[w][r] == -CUDART_INF_F ? 0.f : __expf(sm_m[w][r] - M); Lsum += f[w] * sm_l[w][r]; }
        const uint32_t head = kv * REP + r;
        for (int d = threadIdx.x; d < dh; d += 128) {
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) o += f[w] * sm_acc[w][r][d];
            part[((size_t)split * H + head) * dh + d] = o;
        }
        if (threadIdx.x == 0) { stat[((size_t)split * H + head) * 2] = M; stat[((size_t)split * H + head) * 2 + 1] = Lsum; }
    }

    // ---- the CTA that arrives last at this KV head merges the splits
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(&counters[kv], 1u);
        sm_last = prev == nsplit - 1;
        if (sm_last) counters[kv] = 0u;                       // re-armed for the next launch
    }
    __syncthreads();
    if (tr) { tr[5] = now_ns(); tr[3] = tr[5]; }
    if (!sm_last) return;
    __threadfence();
    // statistics of every (head, split) into shared memory with one load each, then the weights
    float* cm = &sm_acc[0][0][0];                              // [REP][nsplit] max, reused as the split weight
    float* cl = cm + REP * kMaxSplits;                         // [REP][nsplit] sum
    for (uint32_t i = threadIdx.x; i < REP * nsplit; i += 128) {
        const uint32_t r = i / nsplit, s2 = i % nsplit;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(stat + ((size_t)s2 * H + kv * REP + r) * 2));
        cm[r * kMaxSplits + s2] = ml.x; cl[r * kMaxSplits + s2] = ml.y;
    }
    __syncthreads();
    if (threadIdx.x < REP) {
        const uint32_t r = threadIdx.x;
        float M = -CUDART_INF_F, L = 0.f;
        for (uint32_t s2 = 0; s2 < nsplit; ++s2) M = fmaxf(M, cm[r * kMaxSplits + s2]);
        for (uint32_t s2 = 0; s2 < nsplit; ++s2) {
            const float ms = cm[r * kMaxSplits + s2];
            const float wgt = ms == -CUDART_INF_F ? 0.f : __expf(ms - M);
            L += wgt * cl[r * kMaxSplits + s2];
            cm[r * kMaxSplits + s2] = wgt;
        }
        sm_l[0][r] = 1.0f / L;
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < REP * (uint32_t)dh; i += 128) {
        const uint32_t r = i / dh, d = i % dh, head = kv * REP + r;
        float o = 0.f;
        for (uint32_t s0 = 0; s0 < nsplit; s0 += 6) {
            float v[6];
#pragma unroll
            for (int k = 0; k < 6; ++k) v[k] = __ldcg(part + ((size_t)min(s0 + k, nsplit - 1) * H + head) * dh + d);
#pragma unroll
            for (int k = 0; k < 6; ++k) o += s0 + k < nsplit ? cm[r * kMaxSplits + s0 + k] * v[k] : 0.f;
        }
        out[(size_t)head * dh + d] = o * sm_l[0][r];
    }
}

unsigned* attn_counters() {
    static unsigned* p = nullptr;
    if (!p) {
        if (cudaMalloc(&p, 1024 * sizeof(unsigned)) != cudaSuccess) { cudaGetLastError(); p = nullptr; return nullptr; }
        cudaMemset(p, 0, 1024 * sizeof(unsigned));
    }
    return p;
}

template <typename T, int DPL, int REP>
void launch_one(dim3 grid, cudaStream_t st, const float* qkv, void* kc, void* vc, float* part, float* stat, unsigned* counters,
                float* out, unsigned H, unsigned KVH, unsigned ctx, float scale, const float* tbl, unsigned tbl_n, const int* state) {
    static const bool pdl = [] { const char* e = std::getenv("TM_GLUE_PDL"); return !(e && *e == '0'); }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(128); cfg.dynamicSmemBytes = 0; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = pdl ? 1 : 0;
    cudaLaunchKernelEx(&cfg, attn_fused_kernel<T, DPL, REP>, qkv, (T*)kc, (T*)vc, part, stat, counters, out, (uint32_t)H, (uint32_t)KVH,
                       (uint32_t)ctx, scale, (const float2*)tbl, (uint32_t)tbl_n, state, device_trace());
}

template <typename T, int DPL>
bool launch_rep(unsigned REP, dim3 grid, cudaStream_t st, const float* qkv, void* kc, void* vc, float* part, float* stat,
                unsigned* counters, float* out, unsigned H, unsigned KVH, unsigned ctx, float scale, const float* tbl,
                unsigned tbl_n, const int* state) {
    switch (REP) {
        case 1: launch_one<T, DPL, 1>(grid, st, qkv, kc, vc, part, stat, counters, out, H, KVH, ctx, scale, tbl, tbl_n, state); return true;
        case 2: launch_one<T, DPL, 2>(grid, st, qkv, kc, vc, part, stat, counters, out, H, KVH, ctx, scale, tbl, tbl_n, state); return true;
        case 4: launch_one<T, DPL, 4>(grid, st, qkv, kc, vc, part, stat, counters, out, H, KVH, ctx, scale, tbl, tbl_n, state); return true;
        case 8: launch_one<T, DPL, 8>(grid, st, qkv, kc, vc, part, stat, counters, out, H, KVH, ctx, scale, tbl, tbl_n, state); return true;
        default: return fail("attention: REP=%u unsupported (1, 2, 4 or 8)", REP);
    }
}

}  // namespace

unsigned attn_fused_splits(unsigned H, unsigned KVH, unsigned dh, unsigned ctx, size_t scratch_bytes) {
    unsigned nsplit = ((unsigned)device_sm_count() + KVH - 1) / KVH;
    const unsigned tiles = (ctx + 31) / 32;
    if (nsplit > tiles) nsplit = tiles;
    if (nsplit > kMaxSplits) nsplit = kMaxSplits;
    const size_t per_split = (size_t)H * (dh + 2) * sizeof(float);
    const size_t fit = scratch_bytes / per_split;
    if (nsplit > fit) nsplit = (unsigned)fit;
    return nsplit;
}

bool launch_attn_fused(const float* qkv, void* kc, void* vc, bool half_cache, float* scratch, size_t scratch_bytes, float* out,
                       unsigned H, unsigned KVH, unsigned dh, unsigned ctx, float scale, const float* tbl, unsigned tbl_entries,
                       const int* state, cudaStream_t st) {
    if (dh != 64 && dh != 128) return fail("attention: head dim %u unsupported (64 or 128)", dh);
    if (!H || !KVH || H % KVH || KVH > 1024) return fail("attention: bad head counts");
    const unsigned nsplit = attn_fused_splits(H, KVH, dh, ctx, scratch_bytes);
    if (!nsplit) return fail("attention: scratch too small for one split");
    unsigned* counters = attn_counters();
    if (!counters) return fail("attention: counter allocation failed");
    float* part = scratch;
    float* stat = scratch + (size_t)nsplit * H * dh;
    const dim3 grid(KVH, nsplit);
    const unsigned REP = H / KVH;
    bool ok;
    if (half_cache) ok = dh == 128 ? launch_rep<__half, 4>(REP, grid, st, qkv, kc, vc, part, stat, counters, out, H, KVH, ctx, scale, tbl, tbl_entries, state)
                                   : launch_rep<__half, 2>(REP, grid, st, qkv, kc, vc, part, stat, counters, out, H, KVH, ctx, scale, tbl, tbl_entries, state);
    else ok = dh == 128 ? launch_rep<float, 4>(REP, grid, st, qkv, kc, vc, part, stat, counters, out, H, KVH, ctx, scale, tbl, tbl_entries, state)
                        : launch_rep<float, 2>(REP, grid, st, qkv, kc, vc, part, stat, counters, out, H, KVH, ctx, scale, tbl, tbl_entries, state);
    if (!ok) return false;
    note_launch();
    return check_launch("attn_fused");
}

}  // namespace tmc
