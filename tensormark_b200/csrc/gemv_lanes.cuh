// gemv_lanes.cuh — per-lane block decode + dot product of the streaming GEMV.
//
// One warp consumes one "step" of a weight row at a time: a contiguous run of
// blocks staged in shared memory by a bulk copy. Each format fixes how the 32
// lanes divide a step (STEP_W weights, STEP_BYTES bytes), what a lane keeps in
// registers about the activations of its slice (an "x unit" of XW 32-bit words,
// staged once per CTA and reused for every row), and how the lane turns its bytes
// into a partial dot product (dot()).
//
// Arithmetic. The integer codes of a block are never converted one by one. The
// activations of every 32-block are re-expressed once per kernel as block floating
// point: a scale s = max|x|/127 and kPlanes signed 8-bit planes with
//     x[i] ~= s * (a1[i] + a2[i]/128 [+ a3[i]/16384]),
// error <= 2^-15 * max|x| per activation with two planes (the default: 3.1e-5 of the block maximum, which for
// activations of one scale is below 1e-4 * sum|w x| even if every rounding error lined up with the sign of its
// weight, an order inside the 1e-3 contract; measured ~2e-6), <= 2^-22 * max|x| with three (TM_GEMV_PLANES=3
// at build time: the precision of an fp32 product chain, at 1.5x the integer work). A block's dot product is then
// kPlanes exact integer dot products sum(code * a_t) on the dp4a unit (four
// multiply-adds per instruction, the code bytes used as they lie in the block),
// combined in fp32, multiplied by the fp16 block scale and added to the row's fp32
// accumulator: exact within a block, fp32 across blocks, like the reference's
// per-block partial sums (tensormark/llama.h:1877-1895). Zero points and mins are
// applied with the true fp32 sums of x, so nothing depends on the planes' rounding
// beyond the bound above. NaN or infinite activations poison the block scale and
// therefore the output, as a floating-point chain would.
//
// The x planes are laid out to mirror the BYTE positions of the weight block a lane
// reads (scale bytes are matched by zero activation bytes), so a lane never
// realigns or repacks weight words: load, mask nibbles if the format has them,
// dp4a.
//
// Everything here is __host__ __device__: the test-suite replays the lane maps on a
// CPU against the checker before a GPU ever runs them.
//
// Layouts decoded are the serialized blocks of tensormark/quant.h:35-49 and
// 214-245; the GPU kernels replaced are the cooperative-row GEMVs of
// tensormark/metal.h:359-440 (Q4_0), 641-679 (Q4_1), 708-754 (Q5_K), 775-822 (Q6_K).
#pragma once

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#include <cuda_fp16.h>
#define TM_HD __host__ __device__ __forceinline__
#else
#include <math.h>
#define TM_HD inline
struct float2 { float x, y; };
struct float4 { float x, y, z, w; };
struct uint2 { unsigned x, y; };
struct uint4 { unsigned x, y, z, w; };
#endif

namespace tmc {

#ifndef TM_GEMV_PLANES
#define TM_GEMV_PLANES 2
#endif
constexpr int kPlanes = TM_GEMV_PLANES;
static_assert(kPlanes == 2 || kPlanes == 3, "two or three int8 planes");

// ---- primitives with host emulation ----------------------------------------
TM_HD float as_float(uint32_t u) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float f; memcpy(&f, &u, 4); return f;
#endif
}
TM_HD uint32_t as_uint(float f) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    uint32_t u; memcpy(&u, &f, 4); return u;
#endif
}
TM_HD float fma1(float a, float b, float c) {
#if defined(__CUDA_ARCH__)
    return __fmaf_rn(a, b, c);
#else
    return fmaf(a, b, c);
#endif
}
TM_HD float half_to_float(uint32_t h) {
#if defined(__CUDA_ARCH__)
    return __half2float(__ushort_as_half((unsigned short)h));
#else
    const uint32_t s = (h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 1023u;
    if (e == 31u) return as_float(s | 0x7f800000u | (m << 13));
    if (e != 0u) return as_float(s | ((e + 112u) << 23) | (m << 13));
    const float mag = (float)m * 0x1p-24f;
    return as_float(s | as_uint(mag));
#endif
}
TM_HD uint32_t funnel_r(uint32_t lo, uint32_t hi, uint32_t sh) {   // sh in {0, 16}
#if defined(__CUDA_ARCH__)
    return __funnelshift_r(lo, hi, sh);
#else
    return sh ? ((lo >> sh) | (hi << (32 - sh))) : lo;
#endif
}
// c + sum of four (unsigned byte of a) * (signed byte of b)
TM_HD int dp4a_us(uint32_t a, uint32_t b, int c) {
#if defined(__CUDA_ARCH__)
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
#else
    for (int k = 0; k < 4; ++k) c += (int)((a >> (8 * k)) & 0xff) * (int)(int8_t)((b >> (8 * k)) & 0xff);
    return c;
#endif
}
// c + sum of four (signed byte of a) * (signed byte of b)
TM_HD int dp4a_ss(uint32_t a, uint32_t b, int c) {
#if defined(__CUDA_ARCH__)
    return __dp4a((int)a, (int)b, c);
#else
    for (int k = 0; k < 4; ++k) c += (int)(int8_t)((a >> (8 * k)) & 0xff) * (int)(int8_t)((b >> (8 * k)) & 0xff);
    return c;
#endif
}
TM_HD float ld_x(const float* p) {
#if defined(__CUDA_ARCH__)
    return __ldcg(p);           // x is produced by the preceding kernel: read it through L2
#else
    return *p;
#endif
}
TM_HD int round_int(float v) {
#if defined(__CUDA_ARCH__)
    return __float2int_rn(v);
#else
    return (int)lrintf(v);
#endif
}
// S1 + S2/128 [+ S3/16384] in fp32 (each S_t is an exact integer below 2^24)
TM_HD float planes_to_float(const int* S) {
    float f = (float)S[0];
    if (kPlanes > 1) f = fma1((float)S[1], 1.0f / 128.0f, f);
    if (kPlanes > 2) f = fma1((float)S[2], 1.0f / 16384.0f, f);
    return f;
}

// 8 bytes from an address that is 2-byte but maybe not 4-byte aligned.
TM_HD uint2 load8(const uint8_t* p) {
    uint2 r;
#if defined(__CUDA_ARCH__)
    const uint32_t mis = (uint32_t)(uintptr_t)p & 3u;      // 0 or 2
    const uint32_t* a = (const uint32_t*)(p - mis);
    const uint32_t w0 = a[0], w1 = a[1];
    const uint32_t w2 = mis ? a[2] : 0u;
    r.x = funnel_r(w0, w1, mis * 8u);
    r.y = funnel_r(w1, w2, mis * 8u);
#else
    memcpy(&r.x, p, 4); memcpy(&r.y, p + 4, 4);
#endif
    return r;
}
TM_HD uint4 load16a(const void* p) {                       // 16-byte aligned
#if defined(__CUDA_ARCH__)
    return *(const uint4*)p;
#else
    uint4 r; memcpy(&r, p, 16); return r;
#endif
}
TM_HD uint32_t load4a(const uint8_t* p) {
#if defined(__CUDA_ARCH__)
    return *(const uint32_t*)p;
#else
    uint32_t r; memcpy(&r, p, 4); return r;
#endif
}

constexpr uint32_t kLo = 0x0F0F0F0Fu, kHi = 0xF0F0F0F0u;

// ---- block floating point of 32 activations ----------------------------------
// Block scale from the block's max |x| (and whether the block holds NaN/inf):
// x ~= s * (a[0] + a[1]/128 + a[2]/16384). A poisoned block gets s = NaN so every
// output that touches it is NaN; a block of zeros (or of values too small to
// scale) gets s = 0.
TM_HD float block_scale(float amax, bool bad, float& inv) {
    if (bad) { inv = 0.f; return as_float(0x7fc00000u); }
    if (!(amax >= 1.0e-30f)) { inv = 0.f; return 0.f; }
    inv = 127.0f / amax;
    return amax * (1.0f / 127.0f);                          // s * inv == 1 to within 2^-23, far below the plane truncation
}
// The kPlanes signed bytes of one activation under its block's inverse scale: the activation is rounded once to a
// multiple of s / 128^(kPlanes-1) (X = round(v / s * 128^(kPlanes-1))) and X is split into signed digits base 128,
// X = a1 * 16384 + a2 * 128 + a3 (three planes) or a1 * 128 + a2 (two), a1 in [-127, 127], the others in [-64, 64].
// Integer arithmetic after one rounding, which on the GPU is the add of 1.5 * 2^23 (the integer lands in the low
// mantissa bits).
TM_HD void quantize_elem(float v, float inv, int8_t* a) {
    float r = inv == 0.f ? 0.f : v * inv;                   // inv is 0 for empty and for poisoned blocks
    r = r > 127.f ? 127.f : (r < -127.f ? -127.f : r);
    constexpr float kUnit = kPlanes == 3 ? 16384.0f : 128.0f;
#if defined(__CUDA_ARCH__)
    const int X = __float_as_int(__fadd_rn(r * kUnit, 12582912.0f)) - 0x4B400000;
#else
    const int X = (int)lrintf(r * kUnit);
#endif
    if (kPlanes == 3) {
        const int a1 = (X + 8192) >> 14, r1 = X - a1 * 16384;
        const int a2 = (r1 + 64) >> 7, a3 = r1 - a2 * 128;
        a[0] = (int8_t)a1; a[1] = (int8_t)a2; a[kPlanes - 1] = (int8_t)a3;
    } else {
        const int a1 = (X + 64) >> 7, a2 = X - a1 * 128;
        a[0] = (int8_t)a1; a[1] = (int8_t)a2;
    }
}

// two zero bytes at an even byte offset of the x-unit area
TM_HD void zero2(uint32_t* units, uint32_t byte_off) {
    *reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(units) + byte_off) = 0;
}

template <int DT> struct Lane;

// =============================================================================
// 32-weight block formats: a lane owns two consecutive blocks (64 weights) per step;
// an x unit covers the same two blocks.
// =============================================================================

// ---- Q8_0: 34-byte blocks [d:2][q:32], w = q * d --------------------------------
// Lane bytes: 68 = 17 words. Block A's codes sit at unit bytes 2..33, block B's at
// 36..67 (its scale at 34..35). x unit: plane t words [17t, 17t+17) mirror those byte
// positions (zeros under the scale bytes); [17 P] = sA, [17 P + 1] = sB (P = kPlanes).
template <> struct Lane<0> {
    static constexpr int STEP_W = 2048, STEP_BYTES = 2176, UNIT_W = 32, LANE_UNITS = 2, LANE_BYTES = 68;
    static constexpr int SC = 17 * kPlanes;                 // first scalar word
    static constexpr int XW = kPlanes == 3 ? 60 : 36;       // words per x unit; an odd multiple of 4, so 16-byte loads of 8 lanes hit 8 bank groups
    static constexpr bool NEEDS_SUMS = false;               // no zero point, no min: the plain sums of x are not used
    struct X { uint32_t w[XW]; };

    // byte offset, inside the x-unit area, of plane t of activation e
    static TM_HD uint32_t plane_byte(uint32_t e, int t) {
        const uint32_t b = e >> 5, i = e & 31u;
        return (b >> 1) * (XW * 4u) + 68u * (uint32_t)t + ((b & 1u) ? 36u : 2u) + i;
    }
    // plane bytes of four consecutive activations e0..e0+3 (e0 % 4 == 0), packed low byte first
    static TM_HD void store_quad(uint32_t* units, uint32_t e0, int t, uint32_t packed) {
        uint8_t* p = reinterpret_cast<uint8_t*>(units) + plane_byte(e0, t);      // 2 mod 4
        *reinterpret_cast<uint16_t*>(p) = (uint16_t)packed;
        *reinterpret_cast<uint16_t*>(p + 2) = (uint16_t)(packed >> 16);
    }
    // per-32-block scalars; `lane` = first element held by the caller (it passes the sums of the runs that
    // start there), `zl` = the caller's index 0..7 among the threads staging this block
    static TM_HD void scalars(uint32_t* units, uint32_t b, int lane, int zl, float s, float s8, float s16, float s32) {
        (void)s8; (void)s16; (void)s32;
        if (lane == 0) units[(b >> 1) * XW + SC + (b & 1u)] = as_uint(s);
        // the two bytes of every plane image that lie under this block's fp16 scale must read as zero
        if (zl < kPlanes) zero2(units, (b >> 1) * (XW * 4u) + 68u * (uint32_t)zl + ((b & 1u) ? 34u : 0u));
    }
    static TM_HD float dot(const uint8_t* p, const X& x, int lane, int nvalid) {
        (void)lane;
        uint32_t w[17];
#pragma unroll
        for (int i = 0; i < 17; ++i) w[i] = load4a(p + 4 * i);
        int SA[kPlanes], SB[kPlanes];
#pragma unroll
        for (int t = 0; t < kPlanes; ++t) {
            int a = 0, b = 0;
#pragma unroll
            for (int i = 0; i < 9; ++i) a = dp4a_ss(w[i], x.w[17 * t + i], a);
#pragma unroll
            for (int i = 9; i < 17; ++i) b = dp4a_ss(w[i], x.w[17 * t + i], b);
            SA[t] = a; SB[t] = b;
        }
        float acc = half_to_float(w[0] & 0xffffu) * (as_float(x.w[SC]) * planes_to_float(SA));
        if (nvalid > 1) acc = fma1(half_to_float(w[8] >> 16), as_float(x.w[SC + 1]) * planes_to_float(SB), acc);
        return acc;
    }
};

// ---- Q4_0: 18-byte blocks [d:2][qs:16], byte j = elements 2j (low) | 2j+1 (high), w = (n-8)*d
// Lane bytes: 36 = 9 words. x unit: per plane t an "even" 9-word image (element 2j under
// byte j) at [18t, 18t+9) and an "odd" image (element 2j+1) at [18t+9, 18t+18);
// [18 P] = sA, [18 P + 1] = sB, [18 P + 2] = sum(xA), [18 P + 3] = sum(xB) (P = kPlanes).
template <> struct Lane<1> {
    static constexpr int STEP_W = 2048, STEP_BYTES = 1152, UNIT_W = 32, LANE_UNITS = 2, LANE_BYTES = 36;
    static constexpr int SC = 18 * kPlanes;
    static constexpr int XW = kPlanes == 3 ? 60 : 44;
    static constexpr bool NEEDS_SUMS = true;
    struct X { uint32_t w[XW]; };

    static TM_HD uint32_t plane_byte(uint32_t e, int t) {
        const uint32_t b = e >> 5, i = e & 31u;
        return (b >> 1) * (XW * 4u) + 4u * (18u * (uint32_t)t + 9u * (i & 1u)) + ((b & 1u) ? 20u : 2u) + (i >> 1);
    }
    static TM_HD void store_quad(uint32_t* units, uint32_t e0, int t, uint32_t packed) {
        uint8_t* p = reinterpret_cast<uint8_t*>(units) + plane_byte(e0, t);      // even image, even offset
        *reinterpret_cast<uint16_t*>(p) = (uint16_t)((packed & 0xffu) | ((packed >> 8) & 0xff00u));          // elements e0, e0+2
        *reinterpret_cast<uint16_t*>(p + 36) = (uint16_t)(((packed >> 8) & 0xffu) | ((packed >> 16) & 0xff00u));  // e0+1, e0+3
    }
    static TM_HD void scalars(uint32_t* units, uint32_t b, int lane, int zl, float s, float s8, float s16, float s32) {
        (void)s8; (void)s16;
        if (lane == 0) { units[(b >> 1) * XW + SC + (b & 1u)] = as_uint(s); units[(b >> 1) * XW + SC + 2 + (b & 1u)] = as_uint(s32); }
        // zero the bytes under this block's fp16 scale in the even and odd image of every plane
        if (zl < 2 * kPlanes) zero2(units, (b >> 1) * (XW * 4u) + 36u * (uint32_t)zl + ((b & 1u) ? 18u : 0u));
    }
    static TM_HD float dot(const uint8_t* p, const X& x, int lane, int nvalid) {
        (void)lane;
        uint32_t lo[9], hi[9], w0 = 0, w4 = 0;
#pragma unroll
        for (int i = 0; i < 9; ++i) {
            const uint32_t w = load4a(p + 4 * i);
            if (i == 0) w0 = w;
            if (i == 4) w4 = w;
            lo[i] = w & kLo;
            hi[i] = w & kHi;                                 // 16 * high nibble: removed by one shift per block
        }
        int SA[kPlanes], SB[kPlanes];
#pragma unroll
        for (int t = 0; t < kPlanes; ++t) {
            int al = 0, ah = 0, bl = 0, bh = 0;
#pragma unroll
            for (int i = 0; i < 5; ++i) { al = dp4a_us(lo[i], x.w[18 * t + i], al); ah = dp4a_us(hi[i], x.w[18 * t + 9 + i], ah); }
#pragma unroll
            for (int i = 5; i < 9; ++i) { bl = dp4a_us(lo[i], x.w[18 * t + i], bl); bh = dp4a_us(hi[i], x.w[18 * t + 9 + i], bh); }
            SA[t] = al + (ah >> 4);
            SB[t] = bl + (bh >> 4);
        }
        float acc = half_to_float(w0 & 0xffffu) * fma1(as_float(x.w[SC]), planes_to_float(SA), -8.f * as_float(x.w[SC + 2]));
        if (nvalid > 1)
            acc = fma1(half_to_float(w4 >> 16), fma1(as_float(x.w[SC + 1]), planes_to_float(SB), -8.f * as_float(x.w[SC + 3])), acc);
        return acc;
    }
};

// ---- GGUF Q4_0 (dtype 9): the Q4_0 block with split nibbles, byte j = elements j (low) | j + 16 (high)
// (tensormark/llama.h:4588-4597). Same lane bytes, same dot: only the x images differ. The image that meets the
// low nibbles holds element j under byte j, the one that meets the high nibbles element j + 16.
template <> struct Lane<9> : Lane<1> {
    static TM_HD uint32_t plane_byte(uint32_t e, int t) {
        const uint32_t b = e >> 5, i = e & 31u;
        return (b >> 1) * (XW * 4u) + 4u * (18u * (uint32_t)t + 9u * (i >> 4)) + ((b & 1u) ? 20u : 2u) + (i & 15u);
    }
    static TM_HD void store_quad(uint32_t* units, uint32_t e0, int t, uint32_t packed) {
        uint8_t* p = reinterpret_cast<uint8_t*>(units) + plane_byte(e0, t);      // four consecutive bytes of one image, 2 mod 4
        *reinterpret_cast<uint16_t*>(p) = (uint16_t)packed;
        *reinterpret_cast<uint16_t*>(p + 2) = (uint16_t)(packed >> 16);
    }
};

// ---- Q4_1: 20-byte blocks [d:2][m:2][qs:16], byte j = elements j (low) | j+16 (high), w = n*d + m
// Lane bytes: 40 = 10 words. x unit: per block b and plane t a "low" 4-word image at
// [8P b + 8t, +4) and a "high" image at [8P b + 8t + 4, +4); [16 P] = sA, [16 P + 1] = sB,
// [16 P + 2] = sum(xA), [16 P + 3] = sum(xB) (P = kPlanes).
template <> struct Lane<4> {
    static constexpr int STEP_W = 2048, STEP_BYTES = 1280, UNIT_W = 32, LANE_UNITS = 2, LANE_BYTES = 40;
    static constexpr int BW = 8 * kPlanes, SC = 16 * kPlanes;
    static constexpr int XW = kPlanes == 3 ? 52 : 36;
    static constexpr bool NEEDS_SUMS = true;
    struct X { uint32_t w[XW]; };

    static TM_HD uint32_t plane_byte(uint32_t e, int t) {
        const uint32_t b = e >> 5, i = e & 31u;
        return (b >> 1) * (XW * 4u) + 4u * ((uint32_t)BW * (b & 1u) + 8u * (uint32_t)t + 4u * (i >> 4)) + (i & 15u);
    }
    static TM_HD void store_quad(uint32_t* units, uint32_t e0, int t, uint32_t packed) {
        *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(units) + plane_byte(e0, t)) = packed;
    }
    static TM_HD void scalars(uint32_t* units, uint32_t b, int lane, int zl, float s, float s8, float s16, float s32) {
        (void)zl;
        (void)s8; (void)s16;
        if (lane == 0) { units[(b >> 1) * XW + SC + (b & 1u)] = as_uint(s); units[(b >> 1) * XW + SC + 2 + (b & 1u)] = as_uint(s32); }
    }
    template <int B>
    static TM_HD float block(const uint8_t* p, const X& x) {
        const uint32_t hdr = load4a(p + 20 * B);
        uint32_t lo[4], hi[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) { const uint32_t w = load4a(p + 20 * B + 4 + 4 * i); lo[i] = w & kLo; hi[i] = w & kHi; }
        int S[kPlanes];
#pragma unroll
        for (int t = 0; t < kPlanes; ++t) {
            int l = 0, h = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) { l = dp4a_us(lo[i], x.w[BW * B + 8 * t + i], l); h = dp4a_us(hi[i], x.w[BW * B + 8 * t + 4 + i], h); }
            S[t] = l + (h >> 4);
        }
        const float d = half_to_float(hdr & 0xffffu), m = half_to_float(hdr >> 16);
        return fma1(d * as_float(x.w[SC + B]), planes_to_float(S), m * as_float(x.w[SC + 2 + B]));
    }
    static TM_HD float dot(const uint8_t* p, const X& x, int lane, int nvalid) {
        (void)lane;
        float acc = block<0>(p, x);
        if (nvalid > 1) acc += block<1>(p, x);
        return acc;
    }
};

// =============================================================================
// Q5_K: 176-byte super-blocks of 256. Eight lanes share a super-block; lane i takes
// group g = i/2 (64 weights: sub-blocks 2g and 2g+1) and byte half q = i%2: bytes
// 16q..16q+15 of the group's qs, i.e. a run of 16 weights in each sub-block.
// x unit: run0 plane t at [4t, 4t+4), run1 plane t at [4P + 4t, +4); [8 P] = scale of
// sub-block 2g, [8 P + 1] = scale of 2g+1, [8 P + 2] = sum(x run0), [8 P + 3] = sum(x run1) (P = kPlanes).
// =============================================================================
template <> struct Lane<5> {
    static constexpr int STEP_W = 1024, STEP_BYTES = 704, UNIT_W = 256, LANE_UNITS = 1, LANE_BYTES = 0;
    static constexpr int RW = 4 * kPlanes, SC = 8 * kPlanes;
    static constexpr int XW = kPlanes == 3 ? 28 : 20;
    static constexpr bool NEEDS_SUMS = true;
    struct X { uint32_t w[XW]; };

    // 32-block b of the row = sub-block (b % 8) of super-block b / 8; unit = 8*S + 2*g + q
    static TM_HD uint32_t plane_byte(uint32_t e, int t) {
        const uint32_t S = e >> 8, w = e & 255u, g = w >> 6, half = (w >> 5) & 1u, l = w & 31u;
        const uint32_t u = 8u * S + 2u * g + (l >> 4);
        return u * (XW * 4u) + 4u * ((uint32_t)RW * half + 4u * (uint32_t)t) + (l & 15u);
    }
    static TM_HD void store_quad(uint32_t* units, uint32_t e0, int t, uint32_t packed) {
        *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(units) + plane_byte(e0, t)) = packed;
    }
    static TM_HD void scalars(uint32_t* units, uint32_t b, int lane, int zl, float s, float s8, float s16, float s32) {
        (void)zl;
        (void)s8; (void)s32;
        const uint32_t S = b >> 3, j = b & 7u, g = j >> 1, half = j & 1u;
        if ((lane & 15) == 0) {                              // lanes 0 and 16 hold the sums of the two 16-runs
            const uint32_t u = 8u * S + 2u * g + (uint32_t)(lane >> 4);
            units[u * XW + SC + half] = as_uint(s);
            units[u * XW + SC + 2 + half] = as_uint(s16);
        }
    }
    // p: start of the warp's row chunk (16-byte aligned); nvalid: super-blocks present in it
    static TM_HD float dot(const uint8_t* p, const X& x, int lane, int nvalid) {
        const int sb = lane >> 3;
        if (sb >= nvalid) return 0.f;
        const uint32_t g = (uint32_t)(lane & 7) >> 1, q = (uint32_t)lane & 1u;
        const uint8_t* B = p + 176 * sb;
        const uint4 hdr = load16a(B);                       // d|dmin, scales[12]
        const uint4 qh = load16a(B + 16 + 16 * q);
        const uint4 qs = load16a(B + 48 + 32 * g + 16 * q);
        // 6-bit (scale, min) pairs 2g and 2g+1 (quant.h:256-264)
        float sc[2], mn[2];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const uint32_t j = 2u * g + (uint32_t)t, sh = 8u * (j & 3u);
            const uint32_t a = (hdr.y >> sh) & 0xffu, b = (hdr.z >> sh) & 0xffu, c = (hdr.w >> sh) & 0xffu;
            const uint32_t s_lo = a & 63u, m_lo = b & 63u;
            const uint32_t s_hi = (c & 15u) | ((a >> 6) << 4), m_hi = (c >> 4) | ((b >> 6) << 4);
            sc[t] = (float)(j < 4u ? s_lo : s_hi);
            mn[t] = (float)(j < 4u ? m_lo : m_hi);
        }
        const uint32_t wq[4] = {qs.x, qs.y, qs.z, qs.w};
        const uint32_t wh[4] = {qh.x, qh.y, qh.z, qh.w};
        uint32_t c0[4], c1[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t t = wh[e] >> (2u * g);
            c0[e] = (wq[e] & kLo) | ((t << 4) & 0x10101010u);
            c1[e] = ((wq[e] >> 4) & kLo) | ((t << 3) & 0x10101010u);
        }
        int S0[kPlanes], S1[kPlanes];
#pragma unroll
        for (int t = 0; t < kPlanes; ++t) {
            int a = 0, b = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) { a = dp4a_us(c0[e], x.w[4 * t + e], a); b = dp4a_us(c1[e], x.w[RW + 4 * t + e], b); }
            S0[t] = a; S1[t] = b;
        }
        const float d = half_to_float(hdr.x & 0xffffu), dmin = half_to_float(hdr.x >> 16);
        const float pos = fma1(sc[0] * as_float(x.w[SC]), planes_to_float(S0), sc[1] * as_float(x.w[SC + 1]) * planes_to_float(S1));
        const float neg = fma1(mn[0], as_float(x.w[SC + 2]), mn[1] * as_float(x.w[SC + 3]));
        return fma1(d, pos, -(dmin * neg));
    }
};

// =============================================================================
// Q4_K: 144-byte super-blocks of 256 (tensormark/quant.h:222-228, 282-301): the Q5_K block without the
// high bits. Same lane split (eight lanes per super-block, lane i = group i/2, byte half i%2) and the same
// x unit as Q5_K; 16-byte aligned reads because 144 is a multiple of 16.
// =============================================================================
template <> struct Lane<8> : Lane<5> {
    static constexpr int STEP_BYTES = 576;                   // four super-blocks per step
    static TM_HD float dot(const uint8_t* p, const X& x, int lane, int nvalid) {
        const int sb = lane >> 3;
        if (sb >= nvalid) return 0.f;
        const uint32_t g = (uint32_t)(lane & 7) >> 1, q = (uint32_t)lane & 1u;
        const uint8_t* B = p + 144 * sb;
        const uint4 hdr = load16a(B);                       // d|dmin, scales[12]
        const uint4 qs = load16a(B + 16 + 32 * g + 16 * q);
        float sc[2], mn[2];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const uint32_t j = 2u * g + (uint32_t)t, sh = 8u * (j & 3u);
            const uint32_t a = (hdr.y >> sh) & 0xffu, b = (hdr.z >> sh) & 0xffu, c = (hdr.w >> sh) & 0xffu;
            const uint32_t s_lo = a & 63u, m_lo = b & 63u;
            const uint32_t s_hi = (c & 15u) | ((a >> 6) << 4), m_hi = (c >> 4) | ((b >> 6) << 4);
            sc[t] = (float)(j < 4u ? s_lo : s_hi);
            mn[t] = (float)(j < 4u ? m_lo : m_hi);
        }
        const uint32_t wq[4] = {qs.x, qs.y, qs.z, qs.w};
        int S0[kPlanes], S1[kPlanes];
#pragma unroll
        for (int t = 0; t < kPlanes; ++t) {
            int a = 0, b = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) { a = dp4a_us(wq[e] & kLo, x.w[4 * t + e], a); b = dp4a_us((wq[e] >> 4) & kLo, x.w[RW + 4 * t + e], b); }
            S0[t] = a; S1[t] = b;
        }
        const float d = half_to_float(hdr.x & 0xffffu), dmin = half_to_float(hdr.x >> 16);
        const float pos = fma1(sc[0] * as_float(x.w[SC]), planes_to_float(S0), sc[1] * as_float(x.w[SC + 1]) * planes_to_float(S1));
        const float neg = fma1(mn[0], as_float(x.w[SC + 2]), mn[1] * as_float(x.w[SC + 3]));
        return fma1(d, pos, -(dmin * neg));
    }
};

// =============================================================================
// Q6_K: 210-byte super-blocks of 256, only 2-byte aligned. Four lanes share a
// super-block; lane i takes l in [8i, 8i+8) of both 128-halves: for each half 8 bytes
// of ql[l], 8 of ql[l+32], 8 of qh[l] -> 4 runs of 8 weights (elements l + 32j), each
// run inside one 16-weight sub-block with its own int8 scale.
// x unit: run r = 4h + j: plane t words at [2P r + 2t, +2); [16 P + r] = scale of the
// 32-block holding the run, [16 P + 8 + r] = sum(x) over the run (P = kPlanes).
// =============================================================================
template <> struct Lane<6> {
    static constexpr int STEP_W = 2048, STEP_BYTES = 1680, UNIT_W = 256, LANE_UNITS = 1, LANE_BYTES = 0;
    static constexpr int RW = 2 * kPlanes, SC = 16 * kPlanes;
    static constexpr int XW = kPlanes == 3 ? 68 : 52;
    static constexpr bool NEEDS_SUMS = true;
    struct X { uint32_t w[XW]; };

    // 32-block b of the row = run r = b % 8 of super-block b / 8; unit = 4*S + (l / 8)
    static TM_HD uint32_t plane_byte(uint32_t e, int t) {
        const uint32_t S = e >> 8, w = e & 255u, r = w >> 5, l = w & 31u;
        const uint32_t u = 4u * S + (l >> 3);
        return u * (XW * 4u) + 4u * ((uint32_t)RW * r + 2u * (uint32_t)t) + (l & 7u);
    }
    static TM_HD void store_quad(uint32_t* units, uint32_t e0, int t, uint32_t packed) {
        *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(units) + plane_byte(e0, t)) = packed;
    }
    static TM_HD void scalars(uint32_t* units, uint32_t b, int lane, int zl, float s, float s8, float s16, float s32) {
        (void)zl;
        (void)s16; (void)s32;
        const uint32_t S = b >> 3, r = b & 7u;
        if ((lane & 7) == 0) {                               // lanes 0, 8, 16, 24 hold the sums of the four 8-runs
            const uint32_t u = 4u * S + (uint32_t)(lane >> 3);
            units[u * XW + SC + r] = as_uint(s);
            units[u * XW + SC + 8 + r] = as_uint(s8);
        }
    }
    static TM_HD float run_dot(uint32_t c0, uint32_t c1, const X& x, int r, float sc) {
        int S[kPlanes];
#pragma unroll
        for (int t = 0; t < kPlanes; ++t) S[t] = dp4a_us(c1, x.w[RW * r + 2 * t + 1], dp4a_us(c0, x.w[RW * r + 2 * t], 0));
        // codes carry a zero point of 32: sum (c - 32) x = s * S - 32 * sum(x)
        return sc * fma1(as_float(x.w[SC + r]), planes_to_float(S), -32.f * as_float(x.w[SC + 8 + r]));
    }
    static TM_HD float dot(const uint8_t* p, const X& x, int lane, int nvalid) {
        const int sb = lane >> 2;
        if (sb >= nvalid) return 0.f;
        const int i = lane & 3;
        const uint8_t* B = p + 210 * sb;
        float acc = 0.f;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint2 L0 = load8(B + 64 * h + 8 * i);
            const uint2 L1 = load8(B + 64 * h + 32 + 8 * i);
            const uint2 Hh = load8(B + 128 + 32 * h + 8 * i);
            const int8_t* sc = (const int8_t*)(B + 192 + 8 * h + (i >> 1));
            const uint32_t c00 = (L0.x & kLo) | ((Hh.x << 4) & 0x30303030u), c01 = (L0.y & kLo) | ((Hh.y << 4) & 0x30303030u);
            const uint32_t c10 = (L1.x & kLo) | ((Hh.x << 2) & 0x30303030u), c11 = (L1.y & kLo) | ((Hh.y << 2) & 0x30303030u);
            const uint32_t c20 = ((L0.x >> 4) & kLo) | (Hh.x & 0x30303030u), c21 = ((L0.y >> 4) & kLo) | (Hh.y & 0x30303030u);
            const uint32_t c30 = ((L1.x >> 4) & kLo) | ((Hh.x >> 2) & 0x30303030u), c31 = ((L1.y >> 4) & kLo) | ((Hh.y >> 2) & 0x30303030u);
            acc += run_dot(c00, c01, x, 4 * h + 0, (float)sc[0]);
            acc += run_dot(c10, c11, x, 4 * h + 1, (float)sc[2]);
            acc += run_dot(c20, c21, x, 4 * h + 2, (float)sc[4]);
            acc += run_dot(c30, c31, x, 4 * h + 3, (float)sc[6]);
        }
        const uint32_t dh = (uint32_t)B[208] | ((uint32_t)B[209] << 8);
        return half_to_float(dh) * acc;
    }
};

// Copy the lane's x unit from shared memory into registers (16-byte loads).
template <int DT>
TM_HD void load_x_unit(typename Lane<DT>::X& x, const uint32_t* units, uint32_t u) {
    constexpr int XW = Lane<DT>::XW;
    const uint32_t* src = units + (size_t)u * XW;
#pragma unroll
    for (int i = 0; i < XW / 4; ++i) {
        const uint4 v = load16a(src + 4 * i);
        x.w[4 * i] = v.x; x.w[4 * i + 1] = v.y; x.w[4 * i + 2] = v.z; x.w[4 * i + 3] = v.w;
    }
}

}  // namespace tmc
