// llama_stack.cu — the GPU prefill layer stack behind include/llama_gpu_api.h.
//
// CUDA counterpart of the reference's Metal stack (tensormark/metal_llama.h): encode_layer 521-719 (same op order),
// create 727-775, prefill 897-950 and the begin / wait_layer / end form 826-998, with the glue kernels it needs
// (ll_rmsnorm 35-54, ll_rope 61-75, ll_kv_append 78-87, the per-group attention 630-690, ll_silu_mul / ll_add 139-147,
// ll_bias 420-426). The seven projections of a layer are the tensor-core GEMM of gemm.cu; everything between them is
// fp32, which is the reference's "kernel-exactness" mode (bar 1e-3, test_llama_gpu_stack.cpp:10-14).
//
// Where the reference shares the caller's K/V arrays with the GPU through unified memory, this stack keeps fp32 device
// caches [KVH][ctx][dh] per layer, reads rows [0, pos0) from the caller's arrays when a call starts at pos0 > 0, and
// copies the rows it computes back (on a second stream, one event per layer, which is what wait_layer(l) waits for,
// with the reference's 30 s deadline).
//
// Attention: one kernel per layer. A CTA takes one K/V head and a block of query tokens, i.e. 64 query rows
// (tokens x the REP query heads of the group, which share every K/V tile), and walks the keys [0, pos] in tiles of
// 32 with an online softmax. Q K^T and P V are tf32 tensor-core products with fp32 accumulation; scores, softmax
// statistics (one lane per key, warp shuffles) and the running output are fp32.
#include "cuda_shim.h"
#include "llama_gpu_api.h"
#include "common.cuh"
#include "qdecode.cuh"
#include "gemm.h"
#include "glue.h"
#include "state.h"

#include <cuda_fp16.h>

#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <type_traits>
#include <vector>

namespace tmc {
namespace {

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// out[t] = x[t] * rsqrt(mean(x[t]^2) + eps) * w, one CTA per token row (ll_rmsnorm, metal_llama.h:35-54).
// OT = __half: the row goes straight into the next GEMM as its fp16 operand (the same value that GEMM's pre-pass would
// make of the fp32 row: one rounding).
template <typename OT>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                           OT* __restrict__ out, uint32_t D, float eps) {
    __shared__ float part[8];
    __shared__ float inv_s;
    const float* xr = x + (size_t)blockIdx.x * D;
    OT* o = out + (size_t)blockIdx.x * D;
    // rows of up to 8192 values stay in registers between the two passes (16-byte loads, all requested at once)
    constexpr int MAXV = 8;
    const uint32_t n4 = D / 4;
    const bool fits = (D % 4 == 0) && n4 <= 256u * MAXV;
    float4 v[MAXV];
    float p = 0.f;
    if (fits) {
#pragma unroll
        for (int u = 0; u < MAXV; ++u) {
            const uint32_t i = threadIdx.x + u * 256;
            v[u] = i < n4 ? reinterpret_cast<const float4*>(xr)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < MAXV; ++u) { p = fmaf(v[u].x, v[u].x, p); p = fmaf(v[u].y, v[u].y, p); p = fmaf(v[u].z, v[u].z, p); p = fmaf(v[u].w, v[u].w, p); }
    } else {
        for (uint32_t i = threadIdx.x; i < D; i += blockDim.x) { const float t = xr[i]; p = fmaf(t, t, p); }
    }
    p = wsum(p);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = p;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.f;
        for (int i = 0; i < 8; ++i) s += part[i];
        inv_s = 1.0f / sqrtf(s / (float)D + eps);
    }
    __syncthreads();
    const float inv = inv_s;
    if (fits) {
#pragma unroll
        for (int u = 0; u < MAXV; ++u) {
            const uint32_t i = threadIdx.x + u * 256;
            if (i >= n4) continue;
            const float4 ww = reinterpret_cast<const float4*>(w)[i];
            const float a0 = v[u].x * inv * ww.x, a1 = v[u].y * inv * ww.y, a2 = v[u].z * inv * ww.z, a3 = v[u].w * inv * ww.w;
            if constexpr (sizeof(OT) == 2) {
                const __half2 lo = __floats2half2_rn(a0, a1), hi = __floats2half2_rn(a2, a3);
                reinterpret_cast<uint2*>(o)[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
            } else {
                reinterpret_cast<float4*>(o)[i] = make_float4(a0, a1, a2, a3);
            }
        }
    } else {
        for (uint32_t i = threadIdx.x; i < D; i += blockDim.x) {
            const float t = xr[i] * inv * w[i];
            if constexpr (sizeof(OT) == 2) o[i] = __float2half_rn(t); else o[i] = t;
        }
    }
}

// y[t][c] += bias[c] (ll_bias, metal_llama.h:420-426); y rows have stride ld.
__global__ void bias_rows_kernel(float* __restrict__ y, const float* __restrict__ bias, uint32_t n, uint32_t ld, uint32_t T) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)T * n) return;
    const uint32_t t = (uint32_t)(i / n), c = (uint32_t)(i % n);
    y[(size_t)t * ld + c] += bias[c];
}

// For every token t of the batch (position pos0 + t): rotate q in place, rotate k into the K cache row, copy v into the
// V cache row (ll_rope + ll_kv_append, metal_llama.h:61-87; pairs (j, j + dh/2), angles from the shared table).
// kh / vh (both or neither): fp16 copies of the same cache rows, the operands of prefill_attn_h_kernel.
__global__ void rope_append_kernel(float* __restrict__ qkv, uint32_t ld, float* __restrict__ kc, float* __restrict__ vc,
                                   __half* __restrict__ kh, __half* __restrict__ vh,
                                   uint32_t H, uint32_t KVH, uint32_t dh, uint32_t ctx, uint32_t pos0, uint32_t T,
                                   const float2* __restrict__ tbl, uint32_t tbl_n) {
    const uint32_t half = dh / 2, per_tok = (H + KVH) * half + KVH * dh;
    const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (size_t)T * per_tok) return;
    const uint32_t t = (uint32_t)(gid / per_tok), e = (uint32_t)(gid % per_tok), pos = pos0 + t;
    float* row = qkv + (size_t)t * ld;
    if (e < (H + KVH) * half) {
        const uint32_t h = e / half, j = e % half;
        if ((size_t)pos * half + j >= tbl_n) return;
        const float2 cs = tbl[(size_t)pos * half + j];
        float* r = row + (size_t)h * dh;                       // q heads, then k heads, are contiguous in the row
        const float a = r[j], b = r[j + half];
        const float ra = a * cs.x - b * cs.y, rb = b * cs.x + a * cs.y;
        if (h < H) { r[j] = ra; r[j + half] = rb; }
        else {
            const size_t at = ((size_t)(h - H) * ctx + pos) * dh;
            kc[at + j] = ra; kc[at + j + half] = rb;
            if (kh) { kh[at + j] = __float2half_rn(ra); kh[at + j + half] = __float2half_rn(rb); }
        }
    } else {
        const uint32_t i = e - (H + KVH) * half, kv = i / dh, l = i % dh;
        const float v = row[(size_t)(H + KVH) * dh + i];
        vc[((size_t)kv * ctx + pos) * dh + l] = v;
        if (vh) vh[((size_t)kv * ctx + pos) * dh + l] = __float2half_rn(v);
    }
}

__device__ __forceinline__ uint32_t to_tf32(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r;
}
// D += A (16x8, row) * B (8x8, col), tf32 operands, fp32 accumulate.
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Causal GQA attention of a token batch against the fp32 caches. grid (token blocks, KVH), 128 threads = 4 warps.
// Row r of a CTA = token t0 + r / REP, query head g * REP + r % REP; BT = 64 / REP tokens per CTA, keys in tiles of 32.
// Both products run on the tensor cores as m16n8k8 tf32 MMAs with fp32 accumulation: q (pre-scaled), k, v and the
// probabilities are rounded once to tf32 (10 mantissa bits, the precision the projections' fp16 operands have, with
// fp32's range: scores of 128-wide heads overflow fp16); scores, softmax statistics and the output stay fp32.
//
// Warp w owns rows [16 w, +16) for the whole kernel: its q fragments live in registers, the scores of a key tile
// (16 x 32) come out of the MMAs in the accumulator layout - thread (g, t) of a warp holds, per 8 keys, columns 2t and
// 2t + 1 of rows g and g + 8 - and the softmax runs on them in place (row maxima and sums over the four lanes of a
// quad). The probabilities feed the second product without leaving the registers: that product sums over keys, so its
// k index may be any fixed permutation of them, and naming key 2t "k = t" and key 2t + 1 "k = t + 4" makes the
// accumulator layout of P the A-operand layout; V's fragments are loaded with the same naming (rows 2t and 2t + 1).
// K and V tiles arrive by cp.async into a two-deep ring; the thread that copied a piece rounds it to tf32 in place, so
// one barrier publishes a tile and one more protects its buffer from the copy after next: two barriers per 32 keys
// (the previous layout, which split a tile's keys over the warps, took four and sent the scores through shared memory).
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
template <int DH, typename OT>
__global__ void __launch_bounds__(128, 3) prefill_attn_kernel(const float* __restrict__ qkv, uint32_t ld, const float* __restrict__ kc,
                                                              const float* __restrict__ vc, OT* __restrict__ out, uint32_t QD,
                                                              uint32_t T, uint32_t pos0, uint32_t ctx, uint32_t REP, float scale) {
    constexpr int RS = DH + 4;                                  // K and V rows in shared memory: stride 4 (mod 32), conflict-free fragments
    constexpr int D4 = DH / 4;
    constexpr int KS = DH / 8;                                  // k-steps of q k^T
    constexpr int NT = DH / 8;                                  // output n-tiles (a warp holds all DH dims of its rows)
    constexpr int PER = 32 * D4 / 128;                          // 16-byte pieces per thread, tile and tensor
    extern __shared__ __align__(16) float sm[];                 // ring: [buf][K 32 x RS | V 32 x RS]
    const uint32_t BT = 64u / REP, nrows = BT * REP, g = blockIdx.y, t0 = blockIdx.x * BT;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int fg = lane >> 2, ft = lane & 3;
    const uint32_t t_end = min(T, t0 + BT);
    const uint32_t kmax = pos0 + t_end;                         // keys [0, kmax) are visible to the block's last token
    const float* kbase = kc + (size_t)g * ctx * DH;
    const float* vbase = vc + (size_t)g * ctx * DH;

    auto tile_k = [&](int b) { return sm + (size_t)b * 2 * 32 * RS; };
    auto tile_v = [&](int b) { return sm + (size_t)b * 2 * 32 * RS + 32 * RS; };
    auto copy_tile = [&](int b, uint32_t k0) {
        float* Kd = tile_k(b);
        float* Vd = tile_v(b);
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            const int i = tid + u * 128;
            const uint32_t j = i / D4, c = i % D4, kk = k0 + j;
            if (kk < kmax) {
                cp_async16(Kd + j * RS + 4 * c, kbase + (size_t)kk * DH + 4 * c);
                cp_async16(Vd + j * RS + 4 * c, vbase + (size_t)kk * DH + 4 * c);
            } else {
                *reinterpret_cast<float4*>(Kd + j * RS + 4 * c) = make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4*>(Vd + j * RS + 4 * c) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    auto round_own = [&](int b) {                               // the pieces THIS thread copied, fp32 -> tf32 bit patterns
        float* Kd = tile_k(b);
        float* Vd = tile_v(b);
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            const int i = tid + u * 128;
            const uint32_t j = i / D4, c = i % D4;
            const float4 a = *reinterpret_cast<const float4*>(Kd + j * RS + 4 * c), v = *reinterpret_cast<const float4*>(Vd + j * RS + 4 * c);
            uint4 ua, uv;
            ua.x = to_tf32(a.x); ua.y = to_tf32(a.y); ua.z = to_tf32(a.z); ua.w = to_tf32(a.w);
            uv.x = to_tf32(v.x); uv.y = to_tf32(v.y); uv.z = to_tf32(v.z); uv.w = to_tf32(v.w);
            *reinterpret_cast<uint4*>(Kd + j * RS + 4 * c) = ua;
            *reinterpret_cast<uint4*>(Vd + j * RS + 4 * c) = uv;
        }
    };
    copy_tile(0, 0);

    // this lane's rows: r0 = 16 warp + fg and r1 = r0 + 8
    const uint32_t r0 = 16u * warp + fg, r1 = r0 + 8;
    const uint32_t tok0 = t0 + r0 / REP, tok1 = t0 + r1 / REP;
    const bool live0 = r0 < nrows && tok0 < T, live1 = r1 < nrows && tok1 < T;
    // q fragments of the warp's 16 rows, pre-scaled, tf32: a0 (g, t) a1 (g + 8, t) a2 (g, t + 4) a3 (g + 8, t + 4) per k-step
    uint32_t qf[KS][4];
    {
        const float* q0 = qkv + (size_t)(live0 ? tok0 : 0) * ld + (size_t)(g * REP + r0 % REP) * DH;
        const float* q1 = qkv + (size_t)(live1 ? tok1 : 0) * ld + (size_t)(g * REP + r1 % REP) * DH;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qf[ks][0] = to_tf32(live0 ? q0[8 * ks + ft] * scale : 0.f);
            qf[ks][1] = to_tf32(live1 ? q1[8 * ks + ft] * scale : 0.f);
            qf[ks][2] = to_tf32(live0 ? q0[8 * ks + ft + 4] * scale : 0.f);
            qf[ks][3] = to_tf32(live1 ? q1[8 * ks + ft + 4] * scale : 0.f);
        }
    }
    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;    // running maxima (whole row) and this lane's share of the sums
    const uint32_t lim0 = pos0 + tok0, lim1 = pos0 + tok1;      // last visible key of each row

    int buf = 0;
    for (uint32_t k0 = 0; k0 < kmax; k0 += 32, buf ^= 1) {
        if (k0 + 32 < kmax) {
            copy_tile(buf ^ 1, k0 + 32);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        round_own(buf);
        __syncthreads();                                        // tile k0 is in place, rounded
        const uint32_t* Ku = reinterpret_cast<const uint32_t*>(tile_k(buf));
        const uint32_t* Vu = reinterpret_cast<const uint32_t*>(tile_v(buf));
        // scores of the warp's 16 rows x 32 keys: four n-tiles of 8 keys
        float sc[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) sc[j][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                mma_tf32(sc[j], qf[ks], Ku[(8 * j + fg) * RS + 8 * ks + ft], Ku[(8 * j + fg) * RS + 8 * ks + ft + 4]);
        // causal mask, row maxima over the quad
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const uint32_t kk = k0 + 8 * j + 2 * ft + e;
                if (!(live0 && kk <= lim0)) sc[j][e] = -INFINITY;
                if (!(live1 && kk <= lim1)) sc[j][2 + e] = -INFINITY;
                mx0 = fmaxf(mx0, sc[j][e]); mx1 = fmaxf(mx1, sc[j][2 + e]);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        const float al0 = (m0 > -INFINITY) ? expf(m0 - n0) : 1.f, al1 = (m1 > -INFINITY) ? expf(m1 - n1) : 1.f;   // nothing accumulated yet: nothing to rescale
        m0 = n0; m1 = n1;
        uint32_t pf[4][4];                                      // probabilities as A fragments: a0 = (g, key 2t), a2 = (g, key 2t + 1); a1, a3 the same for g + 8
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float p00 = (n0 > -INFINITY) ? expf(sc[j][0] - n0) : 0.f, p01 = (n0 > -INFINITY) ? expf(sc[j][1] - n0) : 0.f;
            const float p10 = (n1 > -INFINITY) ? expf(sc[j][2] - n1) : 0.f, p11 = (n1 > -INFINITY) ? expf(sc[j][3] - n1) : 0.f;
            s0 += p00 + p01; s1 += p10 + p11;
            pf[j][0] = to_tf32(p00); pf[j][2] = to_tf32(p01); pf[j][1] = to_tf32(p10); pf[j][3] = to_tf32(p11);
        }
        l0 = l0 * al0 + s0; l1 = l1 * al1 + s1;
#pragma unroll
        for (int n = 0; n < NT; ++n) { acc[n][0] *= al0; acc[n][1] *= al0; acc[n][2] *= al1; acc[n][3] *= al1; }
        // output += P V, keys 8 j + (2t, 2t + 1) under the names k = t, t + 4
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int n = 0; n < NT; ++n)
                mma_tf32(acc[n], pf[j], Vu[(8 * j + 2 * ft) * RS + 8 * n + fg], Vu[(8 * j + 2 * ft + 1) * RS + 8 * n + fg]);
        __syncthreads();                                        // every warp is done with this buffer: the copy after next may reuse it
    }
    // the lanes of a quad hold disjoint shares of a row's sum
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const bool live = half ? live1 : live0;
        if (!live) continue;
        const uint32_t row = half ? r1 : r0, t = half ? tok1 : tok0;
        const float inv = 1.0f / (half ? l1 : l0);
        OT* o = out + (size_t)t * QD + (size_t)(g * REP + row % REP) * DH + 2 * ft;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            if constexpr (sizeof(OT) == 2) *reinterpret_cast<__half2*>(o + 8 * n) = __floats2half2_rn(acc[n][2 * half] * inv, acc[n][2 * half + 1] * inv);
            else *reinterpret_cast<float2*>(o + 8 * n) = make_float2(acc[n][2 * half] * inv, acc[n][2 * half + 1] * inv);
        }
    }
}

// D += A (16x16, row) * B (16x8, col), fp16 operands, fp32 accumulate.
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// four 8x8 fp16 matrices, row addresses from lanes 8 i .. 8 i + 7; thread (g, t) gets [g][2t, 2t + 1] of each
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const __half* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)) : "memory");
}
// the same, transposed: thread (g, t) gets [2t][g] and [2t + 1][g]
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const __half* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)) : "memory");
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// The same attention over fp16 copies of the cache rows (rope_append_kernel writes them beside the fp32 rows): rows,
// warps and softmax as in prefill_attn_kernel, but both products are m16n8k16 fp16 MMAs with fp32 accumulation - half
// the MMAs per key tile - and the B fragments come out of shared memory by ldmatrix, four 8x8 blocks per instruction
// (K as stored, V transposed), instead of two 32-bit loads per MMA; the tiles need no rounding pass after the copy.
// q (pre-scaled), k, v and the probabilities carry fp16's 10 mantissa bits, as tf32 does; what fp16 lacks is range, and
// a cache value beyond 65504 becomes inf here as it does in the decode lane's fp16 K/V slots. Scores, softmax
// statistics and the output stay fp32. Three 32-key tiles of K and V ride a cp.async ring: one barrier per tile.
template <int DH, typename OT>
__global__ void __launch_bounds__(128, 3) prefill_attn_h_kernel(const float* __restrict__ qkv, uint32_t ld, const __half* __restrict__ kh,
                                                                const __half* __restrict__ vh, OT* __restrict__ out, uint32_t QD,
                                                                uint32_t T, uint32_t pos0, uint32_t ctx, uint32_t REP, float scale) {
    constexpr int RSH = DH + 8;                                 // halves per row in shared memory: 16-byte rows, conflict-free ldmatrix
    constexpr int KS = DH / 16;                                 // k-steps of q k^T
    constexpr int NT = DH / 8;                                  // output n-tiles
    constexpr int NS = 3;                                       // ring depth
    constexpr int C8 = DH / 8;                                  // 16-byte pieces per row
    constexpr int PER = 32 * C8 / 128;                          // pieces per thread, tile and tensor
    extern __shared__ __align__(16) unsigned char sm_raw[];     // ring: [NS][K 32 x RSH | V 32 x RSH] halves
    __half* smh = reinterpret_cast<__half*>(sm_raw);
    const uint32_t BT = 64u / REP, nrows = BT * REP, g = blockIdx.y, t0 = blockIdx.x * BT;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int fg = lane >> 2, ft = lane & 3;
    const uint32_t t_end = min(T, t0 + BT);
    const uint32_t kmax = pos0 + t_end;                         // keys [0, kmax) are visible to the block's last token
    const uint32_t ntiles = (kmax + 31) / 32;
    const __half* kbase = kh + (size_t)g * ctx * DH;
    const __half* vbase = vh + (size_t)g * ctx * DH;

    auto tile_k = [&](int b) { return smh + (size_t)b * 2 * 32 * RSH; };
    auto tile_v = [&](int b) { return smh + (size_t)b * 2 * 32 * RSH + 32 * RSH; };
    auto copy_tile = [&](int b, uint32_t k0) {
        __half* Kd = tile_k(b);
        __half* Vd = tile_v(b);
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            const int i = tid + u * 128;
            const uint32_t j = i / C8, c = i % C8, kk = k0 + j;
            if (kk < kmax) {
                cp_async16(Kd + j * RSH + 8 * c, kbase + (size_t)kk * DH + 8 * c);
                cp_async16(Vd + j * RSH + 8 * c, vbase + (size_t)kk * DH + 8 * c);
            } else {
                *reinterpret_cast<uint4*>(Kd + j * RSH + 8 * c) = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(Vd + j * RSH + 8 * c) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };
#pragma unroll
    for (int s = 0; s < NS - 1; ++s) {                          // one group per ring slot, empty or not: the counts below rely on it
        if ((uint32_t)s < ntiles) copy_tile(s, 32u * s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }

    // this lane's rows: r0 = 16 warp + fg and r1 = r0 + 8
    const uint32_t r0 = 16u * warp + fg, r1 = r0 + 8;
    const uint32_t tok0 = t0 + r0 / REP, tok1 = t0 + r1 / REP;
    const bool live0 = r0 < nrows && tok0 < T, live1 = r1 < nrows && tok1 < T;
    // q fragments of the warp's 16 rows, pre-scaled: a0 (g, 2t..) a1 (g + 8, 2t..) a2 (g, 2t + 8..) a3 (g + 8, 2t + 8..) per k-step
    uint32_t qf[KS][4];
    {
        const float* q0 = qkv + (size_t)(live0 ? tok0 : 0) * ld + (size_t)(g * REP + r0 % REP) * DH + 2 * ft;
        const float* q1 = qkv + (size_t)(live1 ? tok1 : 0) * ld + (size_t)(g * REP + r1 % REP) * DH + 2 * ft;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const float2 a = *reinterpret_cast<const float2*>(q0 + 16 * ks), b = *reinterpret_cast<const float2*>(q1 + 16 * ks);
            const float2 c = *reinterpret_cast<const float2*>(q0 + 16 * ks + 8), d = *reinterpret_cast<const float2*>(q1 + 16 * ks + 8);
            qf[ks][0] = live0 ? pack_h2(a.x * scale, a.y * scale) : 0u;
            qf[ks][1] = live1 ? pack_h2(b.x * scale, b.y * scale) : 0u;
            qf[ks][2] = live0 ? pack_h2(c.x * scale, c.y * scale) : 0u;
            qf[ks][3] = live1 ? pack_h2(d.x * scale, d.y * scale) : 0u;
        }
    }
    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;    // running maxima (whole row) and this lane's share of the sums
    const uint32_t lim0 = pos0 + tok0, lim1 = pos0 + tok1;      // last visible key of each row
    // ldmatrix row of this lane inside a 16 x 16 block: K blocks (keys 0-7 | dims 0-7, 8-15), (keys 8-15 | ...);
    // V blocks (keys 0-7, 8-15 | dims 0-7), (... | dims 8-15)
    const uint32_t k_lane = ((lane >> 4) * 8 + (lane & 7)) * RSH + ((lane >> 3) & 1) * 8;
    const uint32_t v_lane = (((lane >> 3) & 1) * 8 + (lane & 7)) * RSH + (lane >> 4) * 8;

    for (uint32_t it = 0; it < ntiles; ++it) {
        const uint32_t k0 = 32u * it;
        const int buf = (int)(it % NS);
        asm volatile("cp.async.wait_group %0;" ::"n"(NS - 2) : "memory");
        __syncthreads();                                        // tile `it` is in place; every warp is done with tile it - 1
        if (it + NS - 1 < ntiles) copy_tile((int)((it + NS - 1) % NS), k0 + 32u * (NS - 1));
        asm volatile("cp.async.commit_group;" ::: "memory");
        const __half* Kt = tile_k(buf);
        const __half* Vt = tile_v(buf);
        // scores of the warp's 16 rows x 32 keys: four n-tiles of 8 keys
        float sc[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) sc[j][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
#pragma unroll
            for (int jp = 0; jp < 2; ++jp) {
                uint32_t b[4];
                ldsm_x4(b, Kt + 16 * jp * RSH + 16 * ks + k_lane);
                mma_f16(sc[2 * jp], qf[ks], b[0], b[1]);
                mma_f16(sc[2 * jp + 1], qf[ks], b[2], b[3]);
            }
        // causal mask, row maxima over the quad
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const uint32_t kk = k0 + 8 * j + 2 * ft + e;
                if (!(live0 && kk <= lim0)) sc[j][e] = -INFINITY;
                if (!(live1 && kk <= lim1)) sc[j][2 + e] = -INFINITY;
                mx0 = fmaxf(mx0, sc[j][e]); mx1 = fmaxf(mx1, sc[j][2 + e]);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        const float al0 = (m0 > -INFINITY) ? expf(m0 - n0) : 1.f, al1 = (m1 > -INFINITY) ? expf(m1 - n1) : 1.f;   // nothing accumulated yet: nothing to rescale
        m0 = n0; m1 = n1;
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            sc[j][0] = (n0 > -INFINITY) ? expf(sc[j][0] - n0) : 0.f; sc[j][1] = (n0 > -INFINITY) ? expf(sc[j][1] - n0) : 0.f;
            sc[j][2] = (n1 > -INFINITY) ? expf(sc[j][2] - n1) : 0.f; sc[j][3] = (n1 > -INFINITY) ? expf(sc[j][3] - n1) : 0.f;
            s0 += sc[j][0] + sc[j][1]; s1 += sc[j][2] + sc[j][3];
        }
        l0 = l0 * al0 + s0; l1 = l1 * al1 + s1;
#pragma unroll
        for (int n = 0; n < NT; ++n) { acc[n][0] *= al0; acc[n][1] *= al0; acc[n][2] *= al1; acc[n][3] *= al1; }
        // output += P V: the accumulator layout of two 8-key score tiles is the A layout of one 16-key step
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint32_t pf[4];
            pf[0] = pack_h2(sc[2 * i][0], sc[2 * i][1]); pf[1] = pack_h2(sc[2 * i][2], sc[2 * i][3]);
            pf[2] = pack_h2(sc[2 * i + 1][0], sc[2 * i + 1][1]); pf[3] = pack_h2(sc[2 * i + 1][2], sc[2 * i + 1][3]);
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                uint32_t b[4];
                ldsm_x4_t(b, Vt + 16 * i * RSH + 16 * np + v_lane);
                mma_f16(acc[2 * np], pf, b[0], b[1]);
                mma_f16(acc[2 * np + 1], pf, b[2], b[3]);
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // the lanes of a quad hold disjoint shares of a row's sum
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const bool live = half ? live1 : live0;
        if (!live) continue;
        const uint32_t row = half ? r1 : r0, t = half ? tok1 : tok0;
        const float inv = 1.0f / (half ? l1 : l0);
        OT* o = out + (size_t)t * QD + (size_t)(g * REP + row % REP) * DH + 2 * ft;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            if constexpr (sizeof(OT) == 2) *reinterpret_cast<__half2*>(o + 8 * n) = __floats2half2_rn(acc[n][2 * half] * inv, acc[n][2 * half + 1] * inv);
            else *reinterpret_cast<float2*>(o + 8 * n) = make_float2(acc[n][2 * half] * inv, acc[n][2 * half + 1] * inv);
        }
    }
}

// rows [pos0, pos0 + T) of an fp32 cache [KVH][ctx][dh] into a lane K/V slot of the same shape (half or fp32)
template <typename TO>
__global__ void kv_rows_to_slot_kernel(const float* __restrict__ src, TO* __restrict__ dst, uint32_t KVH, uint32_t ctx, uint32_t dh,
                                       uint32_t pos0, uint32_t T) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, per = (size_t)T * dh;
    if (i >= (size_t)KVH * per) return;
    const size_t kv = i / per, off = ((size_t)kv * ctx + pos0) * dh + i % per;
    if constexpr (sizeof(TO) == 2) dst[off] = __float2half_rn(src[off]); else dst[off] = src[off];
}

// rows [pos0, pos0 + T) of the fp16 K and V copies into fp16 lane slots of the same shape, both tensors in one launch
// (blockIdx.y picks one), 16 bytes per thread; dh % 8 == 0
__global__ void kv_half_rows_to_slots_kernel(const uint4* __restrict__ ks, const uint4* __restrict__ vs, uint4* __restrict__ kd, uint4* __restrict__ vd,
                                             uint32_t KVH, uint32_t ctx, uint32_t dh8, uint32_t pos0, uint32_t T) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, per = (size_t)T * dh8;
    if (i >= (size_t)KVH * per) return;
    const size_t off = ((i / per) * ctx + pos0) * dh8 + i % per;
    if (blockIdx.y == 0) kd[off] = ks[off]; else vd[off] = vs[off];
}

struct Layer {
    const uint8_t *q, *k, *v, *o, *gate, *up, *down;            // device block streams
    float *rms1 = nullptr, *rms2 = nullptr, *qb = nullptr, *kb = nullptr, *vb = nullptr;
    float *kc = nullptr, *vc = nullptr;                         // device caches
    __half *kh = nullptr, *vh = nullptr;                        // fp16 copies of their rows, the attention's operands (both or neither)
    // fp16 copies of the static weights (Stack::resident): q|k|v rows stacked [QD + 2 KVD][D], o [D][QD],
    // gate and up rows interleaved [2 F][D] (row 2f = gate f, row 2f + 1 = up f), down [D][F]
    void *wqkv = nullptr, *wo = nullptr, *wgu = nullptr, *wdown = nullptr;
    float *kc_host = nullptr, *vc_host = nullptr;               // the caller's arrays
    bool pinned_k = false, pinned_v = false;
    cudaEvent_t kv_ready = nullptr, kv_done = nullptr;
};
struct Stack {
    int L = 0, D = 0, H = 0, KVH = 0, dh = 0, F = 0, ctx = 0, REP = 0, QD = 0, KVD = 0;
    float theta = 0.f, eps = 0.f;
    unsigned dtype = DT_Q4_0;
    std::vector<Layer> layers;
    float *x = nullptr, *h = nullptr, *qkv = nullptr, *ao = nullptr, *h2 = nullptr, *g = nullptr, *u = nullptr;
    __half *hh = nullptr, *aoh = nullptr, *acth = nullptr;      // resident form: fp16 activations [T][D], [T][QD], [T][F]
    bool resident = false;                                      // the layers hold fp16 copies of their weights
    void* ws = nullptr;
    size_t ws_bytes = 0;
    int cap_T = 0;
    cudaStream_t copy = nullptr;
    cudaEvent_t t0 = nullptr, t1 = nullptr;
    ~Stack() {
        State& s = state();
        if (s.ready) cudaStreamSynchronize(s.stream);
        if (copy) { cudaStreamSynchronize(copy); cudaStreamDestroy(copy); }
        for (Layer& l : layers) {
            for (float* p : {l.rms1, l.rms2, l.qb, l.kb, l.vb, l.kc, l.vc}) if (p) cudaFree(p);
            for (void* p : {l.wqkv, l.wo, l.wgu, l.wdown, (void*)l.kh, (void*)l.vh}) if (p) cudaFree(p);
            if (l.pinned_k) cudaHostUnregister(l.kc_host);
            if (l.pinned_v) cudaHostUnregister(l.vc_host);
            if (l.kv_ready) cudaEventDestroy(l.kv_ready);
            if (l.kv_done) cudaEventDestroy(l.kv_done);
        }
        free_scratch();
        if (t0) cudaEventDestroy(t0);
        if (t1) cudaEventDestroy(t1);
        cudaGetLastError();
    }
    void free_scratch() {
        for (float** p : {&x, &h, &qkv, &ao, &h2, &g, &u}) if (*p) { cudaFree(*p); *p = nullptr; }
        for (__half** p : {&hh, &aoh, &acth}) if (*p) { cudaFree(*p); *p = nullptr; }
        if (ws) { cudaFree(ws); ws = nullptr; }
        cap_T = 0;
    }
};

// the prefill in flight between begin and end (one at a time, like the reference's single shared event)
struct Live { Stack* c = nullptr; int n = 0; bool failed = false; } g_live;
double g_gpu_ms = 0.0;

float* dev_copy(const float* host, size_t n) {
    float* d = nullptr;
    if (cudaMalloc(&d, n * 4) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    if (cudaMemcpy(d, host, n * 4, cudaMemcpyHostToDevice) != cudaSuccess) { cudaGetLastError(); cudaFree(d); return nullptr; }
    return d;
}

bool ensure_scratch(Stack& c, int T) {
    if (T <= c.cap_T) return true;
    State& s = state();
    cudaStreamSynchronize(s.stream);
    c.free_scratch();
    auto mk = [&](size_t floats) { float* p = nullptr; if (cudaMalloc(&p, floats * 4) != cudaSuccess) { cudaGetLastError(); p = nullptr; } return p; };
    const size_t t = (size_t)T;
    auto mkh = [&](size_t halves) { __half* p = nullptr; if (cudaMalloc(&p, halves * 2) != cudaSuccess) { cudaGetLastError(); p = nullptr; } return p; };
    c.x = mk(t * c.D); c.qkv = mk(t * (c.QD + 2 * c.KVD));
    bool ok;
    if (c.resident) {
        if ((c.F % 4) || (c.D % 8) || (c.QD % 8)) return fail("llama stack: row widths must be multiples of 8 (F of 4) for the fp16 activations");
        c.hh = mkh(t * c.D); c.aoh = mkh(t * c.QD); c.acth = mkh(t * c.F);
        ok = c.x && c.qkv && c.hh && c.aoh && c.acth;
    } else {
        c.h = mk(t * c.D); c.h2 = mk(t * c.D); c.ao = mk(t * c.QD); c.g = mk(t * c.F); c.u = mk(t * c.F);
        size_t need = 0;
        for (auto nk : {std::pair<int, int>{c.QD, c.D}, {c.KVD, c.D}, {c.D, c.QD}, {c.F, c.D}, {c.D, c.F}})
            need = std::max(need, gemm_workspace_bytes((unsigned)T, (unsigned)nk.first, (unsigned)nk.second));
        if (cudaMalloc(&c.ws, need) != cudaSuccess) { cudaGetLastError(); c.ws = nullptr; }
        c.ws_bytes = need;
        ok = c.x && c.qkv && c.h && c.h2 && c.ao && c.g && c.u && c.ws;
    }
    if (!ok) { c.free_scratch(); return fail("llama stack: out of device memory for a %d-token batch", T); }
    c.cap_T = T;
    return true;
}

template <int DH> constexpr size_t attn_smem() { return (size_t)(2 * 2 * 32 * (DH + 4)) * 4; }     // two tiles of K and V
template <int DH, typename OT>
bool attn_ready() {
    constexpr size_t smem = attn_smem<DH>();
    static bool attr = false;
    if (!attr) {
        if (cudaFuncSetAttribute(prefill_attn_kernel<DH, OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return fail("llama stack: cannot raise the attention kernel's shared memory limit");
        attr = true;
    }
    return true;
}

template <int DH> constexpr size_t attn_h_smem() { return (size_t)(3 * 2 * 32 * (DH + 8)) * 2; }   // three tiles of K and V, fp16
template <int DH, typename OT>
bool attn_h_ready() {
    static bool attr = false;
    if (!attr) {
        if (cudaFuncSetAttribute(prefill_attn_h_kernel<DH, OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_h_smem<DH>()) != cudaSuccess)
            return fail("llama stack: cannot raise the attention kernel's shared memory limit");
        attr = true;
    }
    return true;
}

bool encode_layer(Stack& c, int l, int T, int pos0, cudaStream_t st) {
    Layer& L = c.layers[(size_t)l];
    const unsigned D = (unsigned)c.D, QD = (unsigned)c.QD, KVD = (unsigned)c.KVD, F = (unsigned)c.F, dh = (unsigned)c.dh;
    const unsigned ld = QD + 2 * KVD, Tn = (unsigned)T;
    const float scale = 1.0f / std::sqrt((float)dh);
    auto gemm = [&](const float* A, const uint8_t* W, float* Cm, unsigned ldc, unsigned N, unsigned K) {
        return launch_gemm(A, W, Cm, ldc, Tn, N, K, c.dtype, c.ws, c.ws_bytes, st);
    };
    auto gemm_h = [&](const __half* Ah, const void* Wh, float* Cm, unsigned ldc, unsigned N, unsigned K, bool accumulate) {
        return launch_gemm_hh(Ah, Wh, Cm, ldc, Tn, N, K, accumulate, st);
    };
    // 1. norm, q / k / v into one [T][QD + 2 KVD] buffer
    if (c.resident) rmsnorm_rows_kernel<__half><<<Tn, 256, 0, st>>>(c.x, L.rms1, c.hh, D, c.eps);
    else rmsnorm_rows_kernel<float><<<Tn, 256, 0, st>>>(c.x, L.rms1, c.h, D, c.eps);
    note_launch();
    if (c.resident) {
        if (!gemm_h(c.hh, L.wqkv, c.qkv, ld, ld, D, false)) return false;            // one GEMM against the stacked rows
    } else if (!gemm(c.h, L.q, c.qkv, ld, QD, D) || !gemm(c.h, L.k, c.qkv + QD, ld, KVD, D) || !gemm(c.h, L.v, c.qkv + QD + KVD, ld, KVD, D)) {
        return false;
    }
    if (L.qb) {
        bias_rows_kernel<<<(unsigned)(((size_t)T * QD + 255) / 256), 256, 0, st>>>(c.qkv, L.qb, QD, ld, Tn);
        bias_rows_kernel<<<(unsigned)(((size_t)T * KVD + 255) / 256), 256, 0, st>>>(c.qkv + QD, L.kb, KVD, ld, Tn);
        bias_rows_kernel<<<(unsigned)(((size_t)T * KVD + 255) / 256), 256, 0, st>>>(c.qkv + QD + KVD, L.vb, KVD, ld, Tn);
        note_launch(3);
    }
    // 2. rope + K/V rows into the caches; the rows then travel to the caller's arrays on the copy stream
    unsigned tbl_n = 0;
    const float* tbl = lane_rope_table(dh, (unsigned)(pos0 + T), c.theta, &tbl_n);
    if (!tbl) return false;
    const size_t per_tok = (size_t)(c.H + c.KVH) * (dh / 2) + (size_t)c.KVH * dh;
    rope_append_kernel<<<(unsigned)(((size_t)T * per_tok + 255) / 256), 256, 0, st>>>(c.qkv, ld, L.kc, L.vc, L.kh, L.vh, (unsigned)c.H, (unsigned)c.KVH, dh,
                                                                                     (unsigned)c.ctx, (unsigned)pos0, Tn, (const float2*)tbl, tbl_n);
    note_launch();
    cudaEventRecord(L.kv_ready, st);
    cudaStreamWaitEvent(c.copy, L.kv_ready, 0);
    if (L.kc_host) {
        const size_t pitch = (size_t)c.ctx * dh * 4, width = (size_t)T * dh * 4, first = (size_t)pos0 * dh;
        cudaMemcpy2DAsync(L.kc_host + first, pitch, L.kc + first, pitch, width, (size_t)c.KVH, cudaMemcpyDeviceToHost, c.copy);
        cudaMemcpy2DAsync(L.vc_host + first, pitch, L.vc + first, pitch, width, (size_t)c.KVH, cudaMemcpyDeviceToHost, c.copy);
    }
    cudaEventRecord(L.kv_done, c.copy);
    // 3. causal attention of the batch over [0, pos]
    const unsigned BT = 64u / (unsigned)c.REP;
    const dim3 grid((Tn + BT - 1) / BT, (unsigned)c.KVH);
    auto attend = [&](auto dhc, auto* dst) -> bool {
        constexpr int DHC = decltype(dhc)::value;
        using OT = std::remove_pointer_t<decltype(dst)>;
        if (L.kh) {
            if (!attn_h_ready<DHC, OT>()) return false;
            prefill_attn_h_kernel<DHC, OT><<<grid, 128, attn_h_smem<DHC>(), st>>>(c.qkv, ld, L.kh, L.vh, dst, QD, Tn, (unsigned)pos0, (unsigned)c.ctx, (unsigned)c.REP, scale);
            return true;
        }
        if (!attn_ready<DHC, OT>()) return false;
        prefill_attn_kernel<DHC, OT><<<grid, 128, attn_smem<DHC>(), st>>>(c.qkv, ld, L.kc, L.vc, dst, QD, Tn, (unsigned)pos0, (unsigned)c.ctx, (unsigned)c.REP, scale);
        return true;
    };
    using I128 = std::integral_constant<int, 128>; using I64 = std::integral_constant<int, 64>;
    if (!(dh == 128 ? (c.resident ? attend(I128{}, c.aoh) : attend(I128{}, c.ao)) : (c.resident ? attend(I64{}, c.aoh) : attend(I64{}, c.ao)))) return false;
    note_launch();
    // 4. o + residual, norm, gate / up, silu * up, down + residual
    if (c.resident) {
        // activations travel as fp16 between the kernels that make them and the GEMMs that read them (one rounding, the
        // one the GEMM's pre-pass would apply), and the residual adds are the GEMMs' own epilogues
        if (!gemm_h(c.aoh, L.wo, c.x, D, D, QD, true)) return false;
        rmsnorm_rows_kernel<__half><<<Tn, 256, 0, st>>>(c.x, L.rms2, c.hh, D, c.eps); note_launch();
        // gate and up rows are interleaved in wgu: one GEMM whose epilogue writes silu(gate) * up as the fp16 operand
        if (!launch_gemm_hh_silu_mul(c.hh, L.wgu, c.acth, Tn, F, D, st)) return false;
        if (!gemm_h(c.acth, L.wdown, c.x, D, D, F, true)) return false;
    } else {
        if (!gemm(c.ao, L.o, c.h2, D, D, QD)) return false;
        if (!launch_add(c.x, c.h2, Tn * D, st)) return false;
        rmsnorm_rows_kernel<float><<<Tn, 256, 0, st>>>(c.x, L.rms2, c.h, D, c.eps); note_launch();
        if (!gemm(c.h, L.gate, c.g, F, F, D) || !gemm(c.h, L.up, c.u, F, F, D)) return false;
        if (!launch_silu_mul(c.g, c.u, Tn * F, st)) return false;
        if (!gemm(c.g, L.down, c.h2, D, D, F)) return false;
        if (!launch_add(c.x, c.h2, Tn * D, st)) return false;
    }
    return check_launch("llama stack layer");
}

// x[t] = row toks[t] of a block-quantized embedding table, dequantized exactly (the decode lane's embed op for a batch)
__global__ void embed_rows_kernel(const int* __restrict__ toks, const uint8_t* __restrict__ W, float* __restrict__ x, uint32_t D,
                                  uint32_t row_bytes, unsigned dtype) {
    const uint32_t k = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (k >= D) return;
    x[(size_t)t * D + k] = decode_weight_dt(dtype, W + (size_t)toks[t] * row_bytes, k);
}

// Where a batch's residual stream comes from: the caller's host rows, or rows of an embedding table on the device.
struct Source { const float* x = nullptr; const int* toks = nullptr; const uint8_t* table = nullptr; unsigned dtype = 0; int vocab = 0; };

// Enqueue the whole batch: x up (or gathered), rows [0, pos0) of the caches up, every layer.
bool enqueue(Stack& c, const Source& src, int T, int pos0) {
    State& s = state();
    if (T < 2 || pos0 < 0 || pos0 + T > c.ctx) return fail("llama stack: batch of %d tokens at position %d does not fit (T >= 2, context %d)", T, pos0, c.ctx);
    if (!src.x && !(src.toks && src.table)) return fail("llama stack: null activations");
    if ((size_t)T * (size_t)c.F > 0xffffffffull) return fail("llama stack: batch too long");
    if (!ensure_scratch(c, T)) return false;
    cudaEventRecord(c.t0, s.stream);
    if (src.x) {
        if (cudaMemcpyAsync(c.x, src.x, (size_t)T * c.D * 4, cudaMemcpyHostToDevice, s.stream) != cudaSuccess) return check_launch("llama stack: x upload");
    } else {
        for (int i = 0; i < T; ++i)
            if (src.toks[i] < 0 || src.toks[i] >= src.vocab) return fail("llama stack: token %d is outside the table of %d rows", src.toks[i], src.vocab);
        // the token ids ride in the tail of the qkv buffer's first row block until the first layer overwrites it
        int* dtoks = reinterpret_cast<int*>(c.qkv);
        if (cudaMemcpyAsync(dtoks, src.toks, (size_t)T * sizeof(int), cudaMemcpyHostToDevice, s.stream) != cudaSuccess) return check_launch("llama stack: token upload");
        const unsigned be = block_elems(src.dtype);
        const uint32_t row_bytes = ((uint32_t)c.D / be) * block_bytes(src.dtype);
        embed_rows_kernel<<<dim3(((unsigned)c.D + 255) / 256, (unsigned)T), 256, 0, s.stream>>>(dtoks, src.table, c.x, (uint32_t)c.D, row_bytes, src.dtype);
        note_launch();
    }
    if (pos0 > 0) {
        // what unified memory would show the reference's GPU: the caller's earlier rows, whoever wrote them
        const size_t pitch = (size_t)c.ctx * c.dh * 4, width = (size_t)pos0 * c.dh * 4;
        for (Layer& L : c.layers) {
            if (!L.kc_host) continue;                               // device-only caches: the earlier rows are where the stack left them
            cudaMemcpy2DAsync(L.kc, pitch, L.kc_host, pitch, width, (size_t)c.KVH, cudaMemcpyHostToDevice, s.stream);
            cudaMemcpy2DAsync(L.vc, pitch, L.vc_host, pitch, width, (size_t)c.KVH, cudaMemcpyHostToDevice, s.stream);
            if (L.kh) {
                const unsigned blocks = (unsigned)(((size_t)c.KVH * pos0 * c.dh + 255) / 256);
                kv_rows_to_slot_kernel<__half><<<blocks, 256, 0, s.stream>>>(L.kc, L.kh, (unsigned)c.KVH, (unsigned)c.ctx, (unsigned)c.dh, 0u, (unsigned)pos0);
                kv_rows_to_slot_kernel<__half><<<blocks, 256, 0, s.stream>>>(L.vc, L.vh, (unsigned)c.KVH, (unsigned)c.ctx, (unsigned)c.dh, 0u, (unsigned)pos0);
                note_launch(2);
            }
        }
        if (!check_launch("llama stack: cache upload")) return false;
    }
    for (int l = 0; l < c.L; ++l)
        if (!encode_layer(c, l, T, pos0, s.stream)) return false;
    cudaEventRecord(c.t1, s.stream);
    return check_launch("llama stack");
}

// Bounded wait for an event (the reference's 30 s deadline, metal_llama.h:856-876).
bool wait_event(cudaEvent_t ev, const char* what) {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(30);
    for (;;) {
        const cudaError_t e = cudaEventQuery(ev);
        if (e == cudaSuccess) return true;
        if (e != cudaErrorNotReady) return fail("llama stack: %s: %s", what, cudaGetErrorString(e));
        if (std::chrono::steady_clock::now() > deadline) return fail("llama stack: %s did not finish within 30 s", what);
    }
}

void* create(const tm_llama_gpu_desc* d, unsigned dtype) {
    if (!d) { fail("llama stack: null description"); return nullptr; }
    if (!ensure_init(-1)) return nullptr;
    if (d->L <= 0 || d->D <= 0 || d->H <= 0 || d->KVH <= 0 || d->F <= 0 || d->ctx <= 0 || !d->layers || d->H % d->KVH || (d->dh & 1) ||
        d->H / d->KVH > 64) { fail("llama stack: invalid dimensions"); return nullptr; }
    if (d->dh != 64 && d->dh != 128) { fail("llama stack: head dimension %d (64 and 128 are built)", d->dh); return nullptr; }
    if (d->D % 4 || (d->H * d->dh) % 4 || (d->KVH * d->dh) % 4) { fail("llama stack: row widths must be multiples of 4"); return nullptr; }
    State& s = state();
    auto c = std::make_unique<Stack>();
    c->L = d->L; c->D = d->D; c->H = d->H; c->KVH = d->KVH; c->dh = d->dh; c->F = d->F; c->ctx = d->ctx;
    c->REP = d->H / d->KVH; c->QD = d->H * d->dh; c->KVD = d->KVH * d->dh; c->theta = d->theta; c->eps = d->eps; c->dtype = dtype;
    if (!weight_bytes(dtype, 1, (size_t)c->D) || !weight_bytes(dtype, 1, (size_t)c->F) || !weight_bytes(dtype, 1, (size_t)c->QD)) {
        fail("llama stack: rows are not whole blocks of dtype %u", dtype); return nullptr;
    }
    if (cudaStreamCreateWithFlags(&c->copy, cudaStreamNonBlocking) != cudaSuccess || cudaEventCreate(&c->t0) != cudaSuccess ||
        cudaEventCreate(&c->t1) != cudaSuccess) { check_launch("llama stack: stream"); return nullptr; }
    c->layers.resize((size_t)c->L);
    const size_t cache_floats = (size_t)c->KVD * c->ctx;
    const char* attn_env = std::getenv("TM_CUDA_STACK_ATTN");
    bool attn_fp16 = !(attn_env && std::strcmp(attn_env, "tf32") == 0);
    for (int l = 0; l < c->L; ++l) {
        const tm_llama_gpu_layer& src = d->layers[l];
        Layer& L = c->layers[(size_t)l];
        // kc and vc both null: the K/V rows stay on the device (tm_cuda_llama_kv_to_slots hands them to the decode lane);
        // the reference, on unified memory, always has the caller's arrays
        if (!src.q || !src.k || !src.v || !src.o || !src.gate || !src.up || !src.down || !src.rms1 || !src.rms2 || (!src.kc != !src.vc)) {
            fail("llama stack: layer %d has a null pointer", l); return nullptr;
        }
        auto reg = [&](const void* p, int rows, int cols) -> const uint8_t* {
            const size_t bytes = weight_bytes(dtype, (size_t)rows, (size_t)cols);
            uint64_t woff = 0;
            const int id = tm_cuda_tok_wbuf(p, bytes, d->map_base, d->map_size, d->map_base ? 1 : 0, &woff);
            return id < 0 ? nullptr : lane_weight_ptr(id, woff, bytes);
        };
        L.q = reg(src.q, c->QD, c->D); L.k = reg(src.k, c->KVD, c->D); L.v = reg(src.v, c->KVD, c->D); L.o = reg(src.o, c->D, c->QD);
        L.gate = reg(src.gate, c->F, c->D); L.up = reg(src.up, c->F, c->D); L.down = reg(src.down, c->D, c->F);
        if (!(L.q && L.k && L.v && L.o && L.gate && L.up && L.down)) return nullptr;
        L.rms1 = dev_copy(src.rms1, (size_t)c->D); L.rms2 = dev_copy(src.rms2, (size_t)c->D);
        if (src.q_bias && src.k_bias && src.v_bias) {
            L.qb = dev_copy(src.q_bias, (size_t)c->QD); L.kb = dev_copy(src.k_bias, (size_t)c->KVD); L.vb = dev_copy(src.v_bias, (size_t)c->KVD);
            if (!(L.qb && L.kb && L.vb)) { fail("llama stack: out of device memory"); return nullptr; }
        }
        if (cudaMalloc(&L.kc, cache_floats * 4) != cudaSuccess || cudaMalloc(&L.vc, cache_floats * 4) != cudaSuccess || !L.rms1 || !L.rms2) {
            cudaGetLastError(); fail("llama stack: out of device memory for the K/V caches"); return nullptr;
        }
        cudaMemsetAsync(L.kc, 0, cache_floats * 4, s.stream); cudaMemsetAsync(L.vc, 0, cache_floats * 4, s.stream);
        // fp16 copies of the rows for the attention's MMAs (half the caches again); TM_CUDA_STACK_ATTN=tf32 does without
        // them and runs the attention on the fp32 rows as tf32, as does a device that has no room for them
        if (attn_fp16) {
            if (cudaMalloc(&L.kh, cache_floats * 2) != cudaSuccess || cudaMalloc(&L.vh, cache_floats * 2) != cudaSuccess) {
                cudaGetLastError();
                for (Layer& M : c->layers) { if (M.kh) cudaFree(M.kh); if (M.vh) cudaFree(M.vh); M.kh = M.vh = nullptr; }
                attn_fp16 = false;
            } else {
                cudaMemsetAsync(L.kh, 0, cache_floats * 2, s.stream); cudaMemsetAsync(L.vh, 0, cache_floats * 2, s.stream);
            }
        }
        L.kc_host = src.kc; L.vc_host = src.vc;
        if (L.kc_host) {
            // page-locking the caller's arrays makes the row copies asynchronous; where it is refused they are staged
            L.pinned_k = cudaHostRegister(L.kc_host, cache_floats * 4, cudaHostRegisterDefault) == cudaSuccess;
            L.pinned_v = cudaHostRegister(L.vc_host, cache_floats * 4, cudaHostRegisterDefault) == cudaSuccess;
            cudaGetLastError();
        }
        if (cudaEventCreateWithFlags(&L.kv_ready, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&L.kv_done, cudaEventDisableTiming) != cudaSuccess) { check_launch("llama stack: events"); return nullptr; }
    }
    // fp16 copies of the weights, made once: 2 bytes per weight of HBM buy every later prefill its weight pre-passes
    // (a quarter of a 512-token prompt's GPU time) and let q|k|v and gate|up run as one GEMM each. Taken when they use
    // no more than a third of the free memory; TM_CUDA_STACK_FP16=0 keeps the per-call conversion, =1 insists.
    {
        const char* e = std::getenv("TM_CUDA_STACK_FP16");
        const int mode = e && *e ? std::atoi(e) : -1;
        const size_t per_layer = 2 * ((size_t)(c->QD + 2 * c->KVD) * c->D + (size_t)c->D * c->QD + (size_t)3 * c->F * c->D);
        size_t free_b = 0, total_b = 0;
        if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) { cudaGetLastError(); free_b = 0; }
        if (mode == 1 || (mode < 0 && per_layer * (size_t)c->L <= free_b / 3)) {
            bool ok = true;
            // gate and up are converted into a staging buffer and copied into alternating rows of wgu
            const size_t row_b = (size_t)c->D * 2;
            void* stage = nullptr;
            ok = cudaMalloc(&stage, (size_t)c->F * row_b) == cudaSuccess;
            for (Layer& L : c->layers) {
                if (!ok) break;
                const size_t qd = (size_t)c->QD * c->D * 2, kvd = (size_t)c->KVD * c->D * 2, fd = (size_t)c->F * c->D * 2;
                ok = ok && cudaMalloc(&L.wqkv, qd + 2 * kvd) == cudaSuccess && cudaMalloc(&L.wo, qd) == cudaSuccess &&
                     cudaMalloc(&L.wgu, 2 * fd) == cudaSuccess && cudaMalloc(&L.wdown, fd) == cudaSuccess;
                if (!ok) break;
                uint8_t* qkv = (uint8_t*)L.wqkv; uint8_t* gu = (uint8_t*)L.wgu;
                ok = launch_weights_f16(L.q, qkv, (unsigned)c->QD, (unsigned)c->D, dtype, s.stream) &&
                     launch_weights_f16(L.k, qkv + qd, (unsigned)c->KVD, (unsigned)c->D, dtype, s.stream) &&
                     launch_weights_f16(L.v, qkv + qd + kvd, (unsigned)c->KVD, (unsigned)c->D, dtype, s.stream) &&
                     launch_weights_f16(L.o, L.wo, (unsigned)c->D, (unsigned)c->QD, dtype, s.stream) &&
                     launch_weights_f16(L.gate, stage, (unsigned)c->F, (unsigned)c->D, dtype, s.stream) &&
                     cudaMemcpy2DAsync(gu, 2 * row_b, stage, row_b, row_b, (size_t)c->F, cudaMemcpyDeviceToDevice, s.stream) == cudaSuccess &&
                     launch_weights_f16(L.up, stage, (unsigned)c->F, (unsigned)c->D, dtype, s.stream) &&
                     cudaMemcpy2DAsync(gu + row_b, 2 * row_b, stage, row_b, row_b, (size_t)c->F, cudaMemcpyDeviceToDevice, s.stream) == cudaSuccess &&
                     launch_weights_f16(L.down, L.wdown, (unsigned)c->D, (unsigned)c->F, dtype, s.stream);
                if (!ok) break;
            }
            if (stage) { cudaStreamSynchronize(s.stream); cudaFree(stage); }
            if (ok) {
                c->resident = true;
            } else {
                cudaGetLastError();
                cudaStreamSynchronize(s.stream);
                for (Layer& L : c->layers)
                    for (void** p : {&L.wqkv, &L.wo, &L.wgu, &L.wdown}) if (*p) { cudaFree(*p); *p = nullptr; }
                if (mode == 1) { fail("llama stack: no room for the fp16 copies of the weights"); return nullptr; }
            }
        }
    }
    if (!sync_stream(s.stream, "llama stack: create")) return nullptr;
    return c.release();
}

}  // namespace
}  // namespace tmc

using namespace tmc;

extern "C" {

void* tm_cuda_llama_create(const tm_llama_gpu_desc* d) { return create(d, DT_Q4_0); }
void* tm_cuda_llama_create_dt(const tm_llama_gpu_desc* d, unsigned dtype) {
    if (!block_elems(dtype) || dtype == DT_F16) { fail("llama stack: dtype %u is not a block format", dtype); return nullptr; }
    return create(d, dtype);
}

void tm_cuda_llama_destroy(void* h) {
    Stack* c = static_cast<Stack*>(h);
    if (g_live.c == c) g_live = Live{};
    delete c;
}

int tm_cuda_llama_prefill_begin(void* h, const float* x, int T, int pos0) {
    Stack* c = static_cast<Stack*>(h);
    if (!c) { fail("llama stack: null handle"); return 0; }
    if (g_live.n) (void)tm_cuda_llama_prefill_end();               // drain an unfinished one, best effort (metal_llama.h:971)
    Source src;
    src.x = x;
    if (!enqueue(*c, src, T, pos0)) return 0;
    g_live.c = c; g_live.n = c->L; g_live.failed = false;
    return 1;
}

int tm_cuda_llama_prefill_begin_tokens(void* h, const int* toks, int T, int pos0, int wid, unsigned long long woff, int vocab, unsigned dtype) {
    Stack* c = static_cast<Stack*>(h);
    if (!c || !toks) { fail("llama stack: null handle or tokens"); return 0; }
    const unsigned be = block_elems(dtype);
    if (!be || dtype == DT_F16 || dtype == DT_BF16 || c->D % (int)be || vocab <= 0) { fail("llama stack: embedding table of dtype %u does not fit rows of %d", dtype, c->D); return 0; }
    Source src;
    src.toks = toks; src.dtype = dtype; src.vocab = vocab;
    src.table = lane_weight_ptr(wid, woff, weight_bytes(dtype, (size_t)vocab, (size_t)c->D));
    if (!src.table) return 0;
    if (g_live.n) (void)tm_cuda_llama_prefill_end();
    if (!enqueue(*c, src, T, pos0)) return 0;
    g_live.c = c; g_live.n = c->L; g_live.failed = false;
    return 1;
}

int tm_cuda_llama_prefill_wait_layer(int l) {
    if (l < 0 || l >= g_live.n || !g_live.c) { fail("llama stack: no layer %d in flight", l); return 0; }
    if (g_live.failed) return 0;
    if (!wait_event(g_live.c->layers[(size_t)l].kv_done, "layer")) { g_live.failed = true; return 0; }
    return 1;
}

int tm_cuda_llama_prefill_end(void) {
    if (!g_live.c || !g_live.n) return 1;
    bool ok = true;
    for (int l = 0; l < g_live.n; ++l)
        if (!tm_cuda_llama_prefill_wait_layer(l)) ok = false;
    State& s = state();
    ok = wait_event(g_live.c->t1, "batch") && ok;
    ok = sync_stream(s.stream, "llama stack") && ok;
    float ms = 0.f;
    if (ok && cudaEventElapsedTime(&ms, g_live.c->t0, g_live.c->t1) == cudaSuccess) g_gpu_ms = ms; else cudaGetLastError();
    g_live.n = 0;
    return ok ? 1 : 0;
}

double tm_cuda_llama_prefill_gpu_ms(void) { return g_gpu_ms; }

int tm_cuda_llama_reserve(void* h, int T) {
    Stack* c = static_cast<Stack*>(h);
    if (!c || T < 2 || T > c->ctx) { fail("llama stack: cannot reserve buffers for %d tokens", T); return 0; }
    return ensure_scratch(*c, T) ? 1 : 0;
}

int tm_cuda_llama_prefill(void* h, float* x, int T, int pos0) {
    Stack* c = static_cast<Stack*>(h);
    if (!c) { fail("llama stack: null handle"); return 0; }
    if (!tm_cuda_llama_prefill_begin(h, x, T, pos0)) return 0;
    State& s = state();
    const bool copied = cudaMemcpyAsync(x, c->x, (size_t)T * c->D * 4, cudaMemcpyDeviceToHost, s.stream) == cudaSuccess;
    const bool ok = tm_cuda_llama_prefill_end() != 0;
    if (!copied) { check_launch("llama stack: x download"); return 0; }
    return ok ? 1 : 0;
}

int tm_cuda_llama_kv_to_slots(void* h, int l, int kcslot, int vcslot, int pos0, int T) {
    Stack* c = static_cast<Stack*>(h);
    if (!c || l < 0 || l >= c->L || pos0 < 0 || T <= 0 || pos0 + T > c->ctx) { fail("llama stack: bad K/V row range"); return 0; }
    State& s = state();
    const size_t elems = (size_t)c->KVD * c->ctx, es = s.kv_half ? 2 : 4;
    uint8_t* kd = lane_slot_ptr(kcslot, elems * es, "llama_kv_to_slots");
    uint8_t* vd = lane_slot_ptr(vcslot, elems * es, "llama_kv_to_slots");
    if (!kd || !vd) return 0;
    const Layer& L = c->layers[(size_t)l];
    const unsigned blocks = (unsigned)(((size_t)c->KVH * T * c->dh + 255) / 256);
    if (s.kv_half && L.kh && c->dh % 8 == 0) {
        // the attention's fp16 rows are the slot's rows already (the same rounding of the same fp32 values)
        const unsigned b8 = (unsigned)(((size_t)c->KVH * T * (c->dh / 8) + 255) / 256);
        kv_half_rows_to_slots_kernel<<<dim3(b8, 2), 256, 0, s.stream>>>((const uint4*)L.kh, (const uint4*)L.vh, (uint4*)kd, (uint4*)vd, (unsigned)c->KVH,
                                                                        (unsigned)c->ctx, (unsigned)c->dh / 8, (unsigned)pos0, (unsigned)T);
        note_launch();
        return check_launch("llama_kv_to_slots") ? 1 : 0;
    }
    if (s.kv_half) {
        kv_rows_to_slot_kernel<__half><<<blocks, 256, 0, s.stream>>>(L.kc, (__half*)kd, (unsigned)c->KVH, (unsigned)c->ctx, (unsigned)c->dh, (unsigned)pos0, (unsigned)T);
        kv_rows_to_slot_kernel<__half><<<blocks, 256, 0, s.stream>>>(L.vc, (__half*)vd, (unsigned)c->KVH, (unsigned)c->ctx, (unsigned)c->dh, (unsigned)pos0, (unsigned)T);
    } else {
        kv_rows_to_slot_kernel<float><<<blocks, 256, 0, s.stream>>>(L.kc, (float*)kd, (unsigned)c->KVH, (unsigned)c->ctx, (unsigned)c->dh, (unsigned)pos0, (unsigned)T);
        kv_rows_to_slot_kernel<float><<<blocks, 256, 0, s.stream>>>(L.vc, (float*)vd, (unsigned)c->KVH, (unsigned)c->ctx, (unsigned)c->dh, (unsigned)pos0, (unsigned)T);
    }
    note_launch(2);
    return check_launch("llama_kv_to_slots") ? 1 : 0;
}

// the reference's names (tensormark/metal_shim.mm:153-160)
void* tm_metal_llama_create(const tm_llama_gpu_desc* d) { return tm_cuda_llama_create(d); }
int tm_metal_llama_prefill(void* h, float* x, int T, int pos0) { return tm_cuda_llama_prefill(h, x, T, pos0); }
int tm_metal_llama_prefill_begin(void* h, const float* x, int T, int pos0) { return tm_cuda_llama_prefill_begin(h, x, T, pos0); }
int tm_metal_llama_prefill_wait_layer(int l) { return tm_cuda_llama_prefill_wait_layer(l); }
int tm_metal_llama_prefill_end(void) { return tm_cuda_llama_prefill_end(); }
double tm_metal_llama_prefill_gpu_ms(void) { return tm_cuda_llama_prefill_gpu_ms(); }
void tm_metal_llama_destroy(void* h) { tm_cuda_llama_destroy(h); }

}  // extern "C"
