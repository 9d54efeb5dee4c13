// glue.cu — the small kernels of the decode chain around the GEMVs.
//
// CUDA forms of the reference's per-token Metal kernels (tensormark/metal.h):
// rmsnorm_row 2408-2434, add_inplace 2444-2449, silu_mul 2450-2455, rope_inplace
// 2460-2475, rope_k_cache(_h) 2478-2508, v_to_cache(_h) 2509-2528, argmax_f32
// 2323-2343, sample_gumbel_f32 2349-2379, embed_q4_row 2380-2395, embed_kq_row
// 1086-1132, tok_bias_qkv 1566-1573, probe_copy 2437-2443, and the GQA split-K
// decode attention attn_decode_gqa(_h) + attn_decode_combine 2739-2859.
// All arithmetic is fp32; K/V rows are rounded to half once, when written.
#include "common.cuh"
#include "glue.h"
#include "exchange.cuh"
#include "qdecode.cuh"

#include <cstdlib>

#include <cuda_fp16.h>
#include <math_constants.h>

namespace tmc {

// Programmatic dependent launch for the chain's small kernels: each one lets its successor become
// resident at once and then waits for its predecessor before it touches any data. A GEMV that
// follows such a kernel is then already on the SMs, pulling its weights, while the small kernel runs.
// Every CTA executes the wait before it can exit, so completion stays transitive along the stream.
// These kernels are resident while their producer still writes, so pointers to produced data carry
// no __restrict__: the compiler must not route those loads through the read-only cache.
__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
template <typename... P, typename... A>
static void launch_pdl(void (*kernel)(P...), dim3 grid, dim3 block, cudaStream_t st, A... args) {
    static const bool on = [] { const char* e = std::getenv("TM_GLUE_PDL"); return !(e && *e == '0'); }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = 0; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = on ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, P(args)...);
}

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// out = x * rsqrt(mean(x^2) + eps) * w; one CTA, two-level reduction
__global__ void __launch_bounds__(1024) rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                        float* __restrict__ out, uint32_t D, float eps) {
    __shared__ float part[32];
    __shared__ float inv_s;
    float p = 0.f;
    for (uint32_t i = threadIdx.x; i < D; i += blockDim.x) { const float v = x[i]; p = fmaf(v, v, p); }
    p = warp_sum(p);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = p;
    __syncthreads();
    if (threadIdx.x < 32) {
        float s = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
        s = warp_sum(s);
        if (threadIdx.x == 0) inv_s = 1.0f / sqrtf(s / (float)D + eps);
    }
    __syncthreads();
    const float inv = inv_s;
    for (uint32_t i = threadIdx.x; i < D; i += blockDim.x) out[i] = x[i] * inv * w[i];
}

__global__ void add_kernel(float* __restrict__ a, const float* __restrict__ b, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] += b[i];
}
__global__ void silu_mul_kernel(float* __restrict__ g, const float* __restrict__ u, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) { const float v = g[i]; g[i] = v / (1.0f + expf(-v)) * u[i]; }
}
__global__ void copy_bytes_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = src[i];
}

// RoPE pairs (j, j + dh/2) from the host-built (cos, sin) table; a position outside
// the table leaves the vector untouched, like the reference kernel.
__global__ void rope_kernel(float* __restrict__ q, uint32_t heads, uint32_t dh, int pos,
                            const float2* __restrict__ tbl, uint32_t tbl_n) {
    const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x, half = dh / 2;
    const uint32_t h = gid / half, j = gid % half;
    if (h >= heads || pos < 0 || (uint32_t)pos * half + j >= tbl_n) return;
    const float2 cs = tbl[(size_t)(uint32_t)pos * half + j];
    float* r = q + (size_t)h * dh;
    const float a = r[j], b = r[j + half];
    r[j] = a * cs.x - b * cs.y;
    r[j + half] = b * cs.x + a * cs.y;
}

template <typename T> __device__ __forceinline__ T to_cache(float v);
template <> __device__ __forceinline__ float to_cache<float>(float v) { return v; }
template <> __device__ __forceinline__ __half to_cache<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__global__ void rope_k_cache_kernel(const float* __restrict__ ksrc, T* __restrict__ cache, uint32_t KVH, uint32_t dh,
                                    uint32_t ctx, int pos, const float2* __restrict__ tbl, uint32_t tbl_n) {
    const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x, half = dh / 2;
    const uint32_t kv = gid / half, j = gid % half;
    if (kv >= KVH || pos < 0 || (uint32_t)pos >= ctx || (uint32_t)pos * half + j >= tbl_n) return;
    const float2 cs = tbl[(size_t)(uint32_t)pos * half + j];
    const float* r = ksrc + (size_t)kv * dh;
    T* dst = cache + (size_t)kv * ctx * dh + (size_t)pos * dh;
    const float a = r[j], b = r[j + half];
    dst[j] = to_cache<T>(a * cs.x - b * cs.y);
    dst[j + half] = to_cache<T>(b * cs.x + a * cs.y);
}
template <typename T>
__global__ void v_cache_kernel(const float* __restrict__ v, T* __restrict__ cache, uint32_t KVH, uint32_t dh,
                               uint32_t ctx, int pos) {
    const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t kv = gid / dh, l = gid % dh;
    if (kv >= KVH || pos < 0 || (uint32_t)pos >= ctx) return;
    cache[(size_t)kv * ctx * dh + (size_t)pos * dh + l] = to_cache<T>(v[gid]);
}
__global__ void f32_to_half_kernel(const float* __restrict__ src, __half* __restrict__ dst, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = __float2half_rn(src[i]);
}
__global__ void half_to_f32_kernel(const __half* __restrict__ src, float* __restrict__ dst, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = __half2float(src[i]);
}

__global__ void bias_kernel(float* __restrict__ y, const float* __restrict__ bias, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] += bias[i];
}

// One embedding row chosen by a token id that lives on the device; the sentinel
// 0xFFFFFFFF (a chain slot not yet written) gives zeros.
// `st` (optional) is a device-resident chain state {position, token index, forced count}: when given, the index comes
// from it; entries below the forced count are prompt tokens that the chooser must not overwrite.
__global__ void embed_row_kernel(const uint32_t* tok, uint32_t idx, const uint8_t* __restrict__ W,
                                 float* x, uint32_t D, uint32_t row_bytes, unsigned dtype,
                                 const int* st) {
    pdl_enter();
    const uint32_t k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= D) return;
    if (st) idx = (uint32_t)st[1];
    const uint32_t row = tok[idx];
    x[k] = row == 0xFFFFFFFFu ? 0.f : decode_weight_dt(dtype, W + (size_t)row * row_bytes, k);
}

// ---- argmax / Gumbel-max over the logits -------------------------------------
// Every CTA reduces a slice to one (value, index) pair packed as a 64-bit key whose
// unsigned order is "larger value first, then lower index"; an atomicMax merges the
// CTAs and the last one to finish publishes the token and re-arms the scratch.
__device__ __forceinline__ unsigned long long pack_key(float v, uint32_t i) {
    uint32_t b = __float_as_uint(v);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);       // monotone map of float order to unsigned order
    return ((unsigned long long)b << 32) | (unsigned long long)(0xFFFFFFFFu - i);
}
__device__ __forceinline__ uint32_t hash32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16; return x;
}

template <bool SAMPLE>
__global__ void __launch_bounds__(256) choose_kernel(const float* x, uint32_t* out, uint32_t n,
                                                      uint32_t idx, float inv_temp, uint32_t seed,
                                                      unsigned long long* scratch /* [0]=key, [1]=done */,
                                                      const int* st, const Exchange xc, int* status) {
    pdl_enter();
    __shared__ unsigned long long best_s[8];
    if (st) {
        idx = (uint32_t)st[1] + 1u;                         // chain: the token chosen now is fed by the next step
        if (idx < (uint32_t)st[2]) return;                  // ... unless that entry is a forced (prompt) token
    }
    exchange_wait(xc, status);                              // sharded head: every rank's slice of x has arrived
    unsigned long long best = pack_key(-CUDART_INF_F, 0);
    const uint32_t base = hash32(seed * 0x9e3779b9u + idx * 0x85ebca6bu + 0x1234567u);
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        float v = __ldcg(x + i);
        if (SAMPLE && inv_temp > 0.f) {
            const uint32_t h = hash32(base ^ (i * 0x27d4eb2fu + 0x165667b1u));
            const float u = ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);
            v = v * inv_temp - logf(-logf(u));
        }
        if (v > -CUDART_INF_F) {                           // NaN and -inf never win, as with `v > best`
            const unsigned long long k = pack_key(v, i);
            best = k > best ? k : best;
        }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const unsigned long long t = __shfl_xor_sync(0xffffffffu, best, o);
        best = t > best ? t : best;
    }
    if ((threadIdx.x & 31) == 0) best_s[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) best = best_s[w] > best ? best_s[w] : best;
        atomicMax(&scratch[0], best);
        __threadfence();
        const unsigned long long done = atomicAdd(&scratch[1], 1ull);
        if (done == gridDim.x - 1) {
            const unsigned long long k = atomicExch(&scratch[0], 0ull);
            scratch[1] = 0ull;
            out[idx] = 0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull);
            __threadfence_system();
        }
    }
}

// The same choice for a row-sharded LM head without gathering the logits: every rank reduces ITS rows [lo, lo + n) of
// x to one key (global row index inside, so the Gumbel noise and the tie rule are those of the unsharded choice), the
// CTA that finishes last stores the key into slot `self` of a small key table here and on every peer, counts itself
// on the site, waits (bounded) for the other ranks' counts and takes the largest of the g keys: g x 8 bytes cross
// NVLink per token instead of the whole vocabulary's logits. A forced (prompt) entry still publishes and counts, so
// that the site's counters keep step with the token epoch, and only leaves the token alone.
template <bool SAMPLE>
__global__ void __launch_bounds__(256) choose_shard_kernel(const float* x, uint32_t* out, uint32_t lo, uint32_t n,
                                                            uint32_t idx, float inv_temp, uint32_t seed,
                                                            unsigned long long* scratch /* [0]=key, [1]=done */,
                                                            const int* st, unsigned long long* keys, const Exchange xc, int* status) {
    pdl_enter();
    __shared__ unsigned long long best_s[8];
    bool forced = false;
    if (st) {
        idx = (uint32_t)st[1] + 1u;
        forced = idx < (uint32_t)st[2];
    }
    unsigned long long best = pack_key(-CUDART_INF_F, 0);
    const uint32_t base = hash32(seed * 0x9e3779b9u + idx * 0x85ebca6bu + 0x1234567u);
    for (uint32_t j = blockIdx.x * blockDim.x + threadIdx.x; j < n; j += gridDim.x * blockDim.x) {
        const uint32_t i = lo + j;
        float v = __ldcg(x + i);
        if (SAMPLE && inv_temp > 0.f) {
            const uint32_t h = hash32(base ^ (i * 0x27d4eb2fu + 0x165667b1u));
            const float u = ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);
            v = v * inv_temp - logf(-logf(u));
        }
        if (v > -CUDART_INF_F) {
            const unsigned long long k = pack_key(v, i);
            best = k > best ? k : best;
        }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const unsigned long long t = __shfl_xor_sync(0xffffffffu, best, o);
        best = t > best ? t : best;
    }
    if ((threadIdx.x & 31) == 0) best_s[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) best = best_s[w] > best ? best_s[w] : best;
        atomicMax(&scratch[0], best);
        __threadfence();
        const unsigned long long done = atomicAdd(&scratch[1], 1ull);
        if (done == gridDim.x - 1) {
            unsigned long long k = atomicExch(&scratch[0], 0ull);
            scratch[1] = 0ull;
            *(volatile unsigned long long*)(keys + xc.self) = k;
            for (uint32_t q = 0; q < xc.npush; ++q) *(volatile unsigned long long*)(reinterpret_cast<unsigned long long*>(xc.peer_y[q]) + xc.self) = k;
            __threadfence_system();                             // the keys before the counts
            for (uint32_t q = 0; q < xc.npush; ++q)
                asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(xc.peer_ctr[q]) : "memory");
            if (exchange_wait_thread(xc, status)) {
                for (uint32_t r = 0; r < xc.nwait; ++r) {
                    if (r == xc.self) continue;
                    const unsigned long long kr = *(volatile const unsigned long long*)(keys + r);
                    k = kr > k ? kr : k;
                }
            }
            if (!forced) {
                out[idx] = 0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull);
                __threadfence_system();
            }
        }
    }
}

// ---- GQA split-K decode attention -------------------------------------------------
// grid (KVH, nsplit), 4 warps. A CTA serves the REP query heads that share one KV
// head over positions [split*chunk, min(allow, (split+1)*chunk)). Each warp walks
// its positions with an online softmax; a lane owns dh/32 consecutive dims, so one
// K or V row is a single coalesced read. The four warps' states are merged in
// shared memory and the CTA writes one unnormalised partial per query head:
// part[(split*H + head)*dh + d] and stat[(split*H + head)*2] = (max, sum).
template <typename T, int DPL, int REP>
__global__ void __launch_bounds__(128) attn_split_kernel(const float* q, const T* kc,
                                                          const T* vc, float* part,
                                                          float* stat, uint32_t H, uint32_t ctx,
                                                          uint32_t allow, uint32_t chunk, float scale,
                                                          const int* st) {
    pdl_enter();
    constexpr int dh = DPL * 32;
    if (st) {                                               // chain: attend [0, position] with the grid's fixed split count
        allow = min((uint32_t)st[0] + 1u, ctx);
        chunk = (allow + gridDim.y - 1) / gridDim.y;
    }
    const uint32_t kv = blockIdx.x, split = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t p0 = split * chunk, p1 = min(allow, p0 + chunk);
    __shared__ float sm_acc[4][REP][dh];
    __shared__ float sm_m[4][REP], sm_l[4][REP];

    float qr[REP][DPL];
#pragma unroll
    for (int r = 0; r < REP; ++r)
#pragma unroll
        for (int d = 0; d < DPL; ++d) qr[r][d] = q[(size_t)(kv * REP + r) * dh + lane * DPL + d] * scale;

    float m[REP], l[REP], acc[REP][DPL];
#pragma unroll
    for (int r = 0; r < REP; ++r) {
        m[r] = -CUDART_INF_F; l[r] = 0.f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[r][d] = 0.f;
    }
    const T* kbase = kc + (size_t)kv * ctx * dh + lane * DPL;
    const T* vbase = vc + (size_t)kv * ctx * dh + lane * DPL;
    for (uint32_t p = p0 + warp; p < p1; p += 4) {
        float kf[DPL], vf[DPL];
#pragma unroll
        for (int d = 0; d < DPL; ++d) { kf[d] = (float)kbase[(size_t)p * dh + d]; vf[d] = (float)vbase[(size_t)p * dh + d]; }
#pragma unroll
        for (int r = 0; r < REP; ++r) {
            float s = 0.f;
#pragma unroll
            for (int d = 0; d < DPL; ++d) s = fmaf(qr[r][d], kf[d], s);
            s = warp_sum(s);
            const float mn = fmaxf(m[r], s);
            const float corr = __expf(m[r] - mn), pw = __expf(s - mn);
            l[r] = l[r] * corr + pw;
#pragma unroll
            for (int d = 0; d < DPL; ++d) acc[r][d] = fmaf(acc[r][d], corr, pw * vf[d]);
            m[r] = mn;
        }
    }
#pragma unroll
    for (int r = 0; r < REP; ++r) {
        if (lane == 0) { sm_m[warp][r] = m[r]; sm_l[warp][r] = l[r]; }
#pragma unroll
        for (int d = 0; d < DPL; ++d) sm_acc[warp][r][lane * DPL + d] = acc[r][d];
    }
    __syncthreads();
    // merge the four warps: thread t handles dims t, t+128, ... of every head
    for (int r = 0; r < REP; ++r) {
        float M = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w][r]);
        float Lsum = 0.f;
        float f[4];
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
}

// out[head][d] = sum_s e^(m_s - M) part_s[d] / sum_s e^(m_s - M) l_s
__global__ void attn_combine_kernel(const float* part, const float* stat, float* out,
                                    uint32_t H, uint32_t dh, uint32_t nsplit) {
    pdl_enter();
    const uint32_t head = blockIdx.x;
    float M = -CUDART_INF_F;
    for (uint32_t s = 0; s < nsplit; ++s) M = fmaxf(M, stat[((size_t)s * H + head) * 2]);
    float L = 0.f;
    for (uint32_t s = 0; s < nsplit; ++s) {
        const float ms = stat[((size_t)s * H + head) * 2];
        if (ms != -CUDART_INF_F) L += __expf(ms - M) * stat[((size_t)s * H + head) * 2 + 1];
    }
    const float invL = 1.0f / L;
    for (uint32_t d = threadIdx.x; d < dh; d += blockDim.x) {
        float o = 0.f;
        for (uint32_t s = 0; s < nsplit; ++s) {
            const float ms = stat[((size_t)s * H + head) * 2];
            if (ms != -CUDART_INF_F) o += __expf(ms - M) * part[((size_t)s * H + head) * dh + d];
        }
        out[(size_t)head * dh + d] = o * invL;
    }
}

// Chain form of rope(q) + rope(k) -> cache + v -> cache in one launch, position read from the chain state.
// qkv = [q: H*dh | k: KVH*dh | v: KVH*dh]; thread t < (H+KVH)*dh/2 rotates one pair, the rest copy V.
template <typename T>
__global__ void qkv_post_kernel(float* qkv, T* kcache, T* vcache, uint32_t H,
                                uint32_t KVH, uint32_t dh, uint32_t ctx, const float2* __restrict__ tbl, uint32_t tbl_n,
                                const int* st) {
    pdl_enter();
    const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x, half = dh / 2;
    const int pos = st[0];
    if (pos < 0 || (uint32_t)pos >= ctx) return;
    const uint32_t npair = (H + KVH) * half;
    if (gid < npair) {
        const uint32_t h = gid / half, j = gid % half;
        if ((uint32_t)pos * half + j >= tbl_n) return;
        const float2 cs = tbl[(size_t)(uint32_t)pos * half + j];
        float* r = qkv + (size_t)h * dh;                     // heads H.. are the K heads, contiguous after q
        const float a = r[j], b = r[j + half];
        const float ra = a * cs.x - b * cs.y, rb = b * cs.x + a * cs.y;
        if (h < H) { r[j] = ra; r[j + half] = rb; }
        else {
            T* dst = kcache + (size_t)(h - H) * ctx * dh + (size_t)pos * dh;
            dst[j] = to_cache<T>(ra); dst[j + half] = to_cache<T>(rb);
        }
    } else if (gid < npair + KVH * dh) {
        const uint32_t e = gid - npair, kv = e / dh, l = e % dh;
        vcache[(size_t)kv * ctx * dh + (size_t)pos * dh + l] = to_cache<T>(qkv[(size_t)(H + KVH) * dh + e]);
    }
}
__global__ void advance_kernel(int* st) { pdl_enter(); st[0] += 1; st[1] += 1; st[3] += 1; }   // position, token index, exchange epoch

inline unsigned cdiv(unsigned a, unsigned b) { return (a + b - 1) / b; }

template <typename T, int DPL>
bool launch_attn_rep(const float* q, const T* kc, const T* vc, float* part, float* stat, unsigned H, unsigned KVH,
                     unsigned ctx, unsigned allow, unsigned chunk, unsigned nsplit, float scale, unsigned REP,
                     const int* state, cudaStream_t st) {
    const dim3 grid(KVH, nsplit);
    switch (REP) {
        case 1: launch_pdl(attn_split_kernel<T, DPL, 1>, grid, dim3(128), st, q, kc, vc, part, stat, H, ctx, allow, chunk, scale, state); break;
        case 2: launch_pdl(attn_split_kernel<T, DPL, 2>, grid, dim3(128), st, q, kc, vc, part, stat, H, ctx, allow, chunk, scale, state); break;
        case 4: launch_pdl(attn_split_kernel<T, DPL, 4>, grid, dim3(128), st, q, kc, vc, part, stat, H, ctx, allow, chunk, scale, state); break;
        case 8: launch_pdl(attn_split_kernel<T, DPL, 8>, grid, dim3(128), st, q, kc, vc, part, stat, H, ctx, allow, chunk, scale, state); break;
        default: return fail("attention: REP=%u unsupported (1, 2, 4 or 8)", REP);
    }
    note_launch();
    return check_launch("attn_split");
}

}  // namespace

bool launch_rmsnorm(const float* x, const float* w, float* out, unsigned D, float eps, cudaStream_t st) {
    if (!x || !w || !out || D == 0) return fail("rmsnorm: bad arguments");
    const unsigned threads = D >= 4096 ? 1024 : D >= 1024 ? 512 : 256;
    rmsnorm_kernel<<<1, threads, 0, st>>>(x, w, out, D, eps);
    note_launch();
    return check_launch("rmsnorm");
}
bool launch_add(float* a, const float* b, unsigned n, cudaStream_t st) {
    if (!a || !b) return fail("add: null pointer");
    if (n == 0) return true;
    add_kernel<<<cdiv(n, 256), 256, 0, st>>>(a, b, n);
    note_launch();
    return check_launch("add");
}
bool launch_silu_mul(float* g, const float* u, unsigned n, cudaStream_t st) {
    if (!g || !u) return fail("silu_mul: null pointer");
    if (n == 0) return true;
    silu_mul_kernel<<<cdiv(n, 256), 256, 0, st>>>(g, u, n);
    note_launch();
    return check_launch("silu_mul");
}
bool launch_bias(float* y, const float* bias, unsigned n, cudaStream_t st) {
    if (!y || !bias) return fail("bias: null pointer");
    if (n == 0) return true;
    bias_kernel<<<cdiv(n, 256), 256, 0, st>>>(y, bias, n);
    note_launch();
    return check_launch("bias");
}
bool launch_copy_bytes(const uint8_t* src, uint8_t* dst, unsigned n, cudaStream_t st) {
    if (n == 0) return true;
    copy_bytes_kernel<<<cdiv(n, 256), 256, 0, st>>>(src, dst, n);
    note_launch();
    return check_launch("probe_copy");
}
bool launch_rope(float* q, unsigned heads, unsigned dh, int pos, const float* tbl, unsigned tbl_entries, cudaStream_t st) {
    const unsigned pairs = heads * (dh / 2);
    if (pairs == 0) return true;
    rope_kernel<<<cdiv(pairs, 128), 128, 0, st>>>(q, heads, dh, pos, (const float2*)tbl, tbl_entries);
    note_launch();
    return check_launch("rope");
}
bool launch_rope_k_cache(const float* ksrc, void* cache, bool half_cache, unsigned KVH, unsigned dh, unsigned ctx, int pos,
                         const float* tbl, unsigned tbl_entries, cudaStream_t st) {
    const unsigned pairs = KVH * (dh / 2);
    if (pairs == 0) return true;
    if (half_cache) rope_k_cache_kernel<__half><<<cdiv(pairs, 128), 128, 0, st>>>(ksrc, (__half*)cache, KVH, dh, ctx, pos, (const float2*)tbl, tbl_entries);
    else rope_k_cache_kernel<float><<<cdiv(pairs, 128), 128, 0, st>>>(ksrc, (float*)cache, KVH, dh, ctx, pos, (const float2*)tbl, tbl_entries);
    note_launch();
    return check_launch("rope_k_cache");
}
bool launch_v_cache(const float* v, void* cache, bool half_cache, unsigned KVH, unsigned dh, unsigned ctx, int pos, cudaStream_t st) {
    const unsigned n = KVH * dh;
    if (n == 0) return true;
    if (half_cache) v_cache_kernel<__half><<<cdiv(n, 128), 128, 0, st>>>(v, (__half*)cache, KVH, dh, ctx, pos);
    else v_cache_kernel<float><<<cdiv(n, 128), 128, 0, st>>>(v, (float*)cache, KVH, dh, ctx, pos);
    note_launch();
    return check_launch("v_cache");
}
bool launch_f32_to_half(const float* src, void* dst, size_t n, cudaStream_t st) {
    if (n == 0) return true;
    f32_to_half_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(src, (__half*)dst, n);
    note_launch();
    return check_launch("f32_to_half");
}
bool launch_half_to_f32(const void* src, float* dst, size_t n, cudaStream_t st) {
    if (n == 0) return true;
    half_to_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>((const __half*)src, dst, n);
    note_launch();
    return check_launch("half_to_f32");
}
bool launch_embed_row(const unsigned* tok, unsigned idx, const uint8_t* W, float* x, unsigned D, unsigned dtype, cudaStream_t st,
                      const int* state) {
    const unsigned be = block_elems(dtype);
    if (!be || dtype == DT_F16 || D % be) return fail("embed: D=%u is not whole blocks of dtype %u", D, dtype);
    launch_pdl(embed_row_kernel, dim3(cdiv(D, 256)), dim3(256), st, tok, idx, W, x, D, (D / be) * block_bytes(dtype), dtype, state);
    note_launch();
    return check_launch("embed_row");
}
bool launch_choose(const float* x, unsigned* out, unsigned n, unsigned idx, float inv_temp, unsigned seed, bool sample,
                   unsigned long long* scratch, cudaStream_t st, const int* state, const Exchange* xchg) {
    if (!x || !out || n == 0) return fail("argmax: bad arguments");
    unsigned grid = cdiv(n, 256 * 4);
    const unsigned sms = (unsigned)device_sm_count();
    if (grid > sms) grid = sms;
    const Exchange xc = xchg ? *xchg : Exchange{};
    if (xc.nwait && (!xc.wait_ctrs || !xc.wait_ctas || !xc.epoch)) return fail("argmax: incomplete peer exchange description");
    if (sample) launch_pdl(choose_kernel<true>, dim3(grid), dim3(256), st, x, out, n, idx, inv_temp, seed, scratch, state, xc, device_status_word());
    else launch_pdl(choose_kernel<false>, dim3(grid), dim3(256), st, x, out, n, idx, 0.f, 0u, scratch, state, xc, device_status_word());
    note_launch();
    return check_launch("argmax");
}

bool launch_choose_shard(const float* x, unsigned* out, unsigned lo, unsigned n, float inv_temp, unsigned seed, bool sample,
                         unsigned long long* scratch, unsigned long long* keys, cudaStream_t st, const int* state, const Exchange& xc) {
    if (!x || !out || !keys || !state || n == 0) return fail("choose_shard: bad arguments");
    if (!xc.nwait || !xc.wait_ctrs || xc.wait_ctas != 1 || !xc.epoch || xc.npush + 1 != xc.nwait)
        return fail("choose_shard: incomplete peer exchange description");
    unsigned grid = cdiv(n, 256 * 4);
    const unsigned sms = (unsigned)device_sm_count();
    if (grid > sms) grid = sms;
    if (sample) launch_pdl(choose_shard_kernel<true>, dim3(grid), dim3(256), st, x, out, lo, n, 0u, inv_temp, seed, scratch, state, keys, xc, device_status_word());
    else launch_pdl(choose_shard_kernel<false>, dim3(grid), dim3(256), st, x, out, lo, n, 0u, 0.f, 0u, scratch, state, keys, xc, device_status_word());
    note_launch();
    return check_launch("choose_shard");
}

bool launch_qkv_post(float* qkv, void* kc, void* vc, bool half_cache, unsigned H, unsigned KVH, unsigned dh, unsigned ctx,
                     const float* tbl, unsigned tbl_entries, const int* state, cudaStream_t st) {
    const unsigned n = (H + KVH) * (dh / 2) + KVH * dh;
    if (half_cache) launch_pdl(qkv_post_kernel<__half>, dim3(cdiv(n, 256)), dim3(256), st, qkv, (__half*)kc, (__half*)vc, H, KVH, dh, ctx, (const float2*)tbl, tbl_entries, state);
    else launch_pdl(qkv_post_kernel<float>, dim3(cdiv(n, 256)), dim3(256), st, qkv, (float*)kc, (float*)vc, H, KVH, dh, ctx, (const float2*)tbl, tbl_entries, state);
    note_launch();
    return check_launch("qkv_post");
}
bool launch_advance(int* state, cudaStream_t st) {
    launch_pdl(advance_kernel, dim3(1), dim3(1), st, state);
    note_launch();
    return check_launch("advance");
}

AttnPlan plan_attention(unsigned H, unsigned KVH, unsigned dh, unsigned ctx, unsigned allow, size_t probs_bytes) {
    return plan_attention_sms((unsigned)device_sm_count(), H, KVH, dh, ctx, allow, probs_bytes);
}
AttnPlan plan_attention_sms(unsigned sms, unsigned H, unsigned KVH, unsigned dh, unsigned ctx, unsigned allow, size_t probs_bytes) {
    AttnPlan pl{};
    // Enough (kv head, split) CTAs to cover the machine; every split at least 32
    // positions; the partials must fit the caller's probs buffer.
    unsigned nsplit = cdiv(sms, KVH);
    nsplit = nsplit < cdiv(allow, 32u) ? nsplit : cdiv(allow, 32u);
    const size_t per_split = (size_t)H * (dh + 2) * sizeof(float);
    const unsigned fit = (unsigned)(probs_bytes / per_split);
    if (fit == 0) { pl.nsplit = 0; return pl; }
    if (nsplit > fit) nsplit = fit;
    if (nsplit == 0) nsplit = 1;
    pl.chunk = cdiv(allow, nsplit);
    pl.nsplit = cdiv(allow, pl.chunk);
    pl.part_floats = (size_t)pl.nsplit * H * dh;
    (void)ctx;
    return pl;
}

bool launch_attention(const float* q, const void* kc, const void* vc, bool half_cache, float* scratch, float* out,
                      unsigned H, unsigned KVH, unsigned dh, unsigned ctx, unsigned allow, float scale, unsigned REP,
                      const AttnPlan& pl, cudaStream_t st, const int* state) {
    if (dh != 64 && dh != 128) return fail("attention: head dim %u unsupported (64 or 128)", dh);
    float* part = scratch;
    float* stat = scratch + pl.part_floats;
    bool ok;
    if (half_cache) {
        ok = dh == 128 ? launch_attn_rep<__half, 4>(q, (const __half*)kc, (const __half*)vc, part, stat, H, KVH, ctx, allow, pl.chunk, pl.nsplit, scale, REP, state, st)
                       : launch_attn_rep<__half, 2>(q, (const __half*)kc, (const __half*)vc, part, stat, H, KVH, ctx, allow, pl.chunk, pl.nsplit, scale, REP, state, st);
    } else {
        ok = dh == 128 ? launch_attn_rep<float, 4>(q, (const float*)kc, (const float*)vc, part, stat, H, KVH, ctx, allow, pl.chunk, pl.nsplit, scale, REP, state, st)
                       : launch_attn_rep<float, 2>(q, (const float*)kc, (const float*)vc, part, stat, H, KVH, ctx, allow, pl.chunk, pl.nsplit, scale, REP, state, st);
    }
    if (!ok) return false;
    launch_pdl(attn_combine_kernel, dim3(H), dim3(dh < 128 ? 64 : 128), st, part, stat, out, H, dh, pl.nsplit);
    note_launch();
    return check_launch("attn_combine");
}

}  // namespace tmc
