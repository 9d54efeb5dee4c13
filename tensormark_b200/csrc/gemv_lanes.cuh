// gemv_lanes.cuh — per-lane block decode + dot product of the streaming GEMV.
//
// One warp consumes one "step" of a weight row at a time: a contiguous run of
// blocks staged in shared memory by a bulk copy. Each format fixes how the 32
// lanes divide a step (STEP_W weights, STEP_BYTES bytes), which activations a
// lane keeps in registers for that step (struct X, loaded once and reused for
// every row of the warp's row group), and how the lane turns its bytes into a
// partial dot product (dot()).
//
// Decoding never converts integers: a code byte is moved by one PRMT into the
// mantissa of a constant (128.0f for codes below 128, 32768.0f for full bytes),
// which yields the float (OFFSET + code) exactly. Products are accumulated with
// packed FFMA2 and the offset (plus the format's zero point) is removed once per
// block with the block's activation sum:  sum (code-zp)*x = sum f*x - (OFF+zp)*X.
// The added rounding error is below 1e-5 of sum|w*x| for every format here,
// against the path's 1e-3 tolerance. Q8_0 bytes would need OFFSET 32768 (~500x
// the mean code), so its offset is subtracted exactly before the multiply.
//
// Everything in this header is __host__ __device__ so the lane maps can be run
// lane by lane on a CPU against the checker before a GPU ever sees them.
//
// Layouts decoded here are the serialized blocks of tensormark/quant.h:35-49 and
// 214-245; the GPU kernels they replace are the cooperative-row GEMVs of
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

// ---- primitives with host emulation ----------------------------------------
TM_HD uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
#if defined(__CUDA_ARCH__)
    return __byte_perm(a, b, sel);
#else
    const uint64_t v = ((uint64_t)b << 32) | a;
    uint32_t r = 0;
    for (int k = 0; k < 4; ++k) r |= (uint32_t)((v >> (8 * ((sel >> (4 * k)) & 7))) & 0xff) << (8 * k);
    return r;
#endif
}
TM_HD float as_float(uint32_t u) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float f; memcpy(&f, &u, 4); return f;
#endif
}
TM_HD float2 fma2(float2 a, float2 b, float2 c) {
#if defined(__CUDA_ARCH__)
    return __ffma2_rn(a, b, c);
#else
    float2 r; r.x = fmaf(a.x, b.x, c.x); r.y = fmaf(a.y, b.y, c.y); return r;
#endif
}
TM_HD float2 add2(float2 a, float2 b) {
#if defined(__CUDA_ARCH__)
    return __fadd2_rn(a, b);
#else
    float2 r; r.x = a.x + b.x; r.y = a.y + b.y; return r;
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
    uint32_t b; memcpy(&b, &mag, 4);
    return as_float(s | b);
#endif
}
TM_HD uint32_t funnel_r(uint32_t lo, uint32_t hi, uint32_t sh) {   // sh in {0, 16}
#if defined(__CUDA_ARCH__)
    return __funnelshift_r(lo, hi, sh);
#else
    return sh ? ((lo >> sh) | (hi << (32 - sh))) : lo;
#endif
}

// float (128 + byte B of a), valid for bytes below 128
template <int B> TM_HD float code128(uint32_t a) { return as_float(prmt(a, 0x43000000u, 0x7054u | (B << 8))); }
// float (32768 + byte B of a), any byte
template <int B> TM_HD float code32768(uint32_t a) { return as_float(prmt(a, 0x47000000u, 0x7604u | (B << 4))); }

// Activations live in shared memory as float4 slots, XOR-swizzled so that the 8
// lanes of a quarter warp that read 64-byte-strided runs hit different banks.
TM_HD uint32_t x_slot(uint32_t q) { return q ^ ((q >> 4) & 7u); }

TM_HD float2 mk2(float a, float b) { float2 r; r.x = a; r.y = b; return r; }

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
TM_HD uint4 load16a(const uint8_t* p) {                    // 16-byte aligned
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

constexpr uint32_t kLo = 0x0F0F0F0Fu;

// ---------------------------------------------------------------------------
// 32-weight block formats: a lane owns two consecutive blocks (64 weights).
// ---------------------------------------------------------------------------
struct X64 {
    float2 v[32];     // the lane's 64 activations, in element order
    float bs[2];      // activation sums of its two 32-blocks
};

// chunk = index of this step inside the row; xs4 = swizzled activations;
// xsum = per-32-block activation sums (zero padded to whole steps).
TM_HD void load_x64(X64& x, const float4* xs4, const float* xsum, int chunk, int lane) {
    const uint32_t q0 = (uint32_t)chunk * 512u + (uint32_t)lane * 16u;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float4 t = xs4[x_slot(q0 + i)];
        x.v[2 * i] = mk2(t.x, t.y);
        x.v[2 * i + 1] = mk2(t.z, t.w);
    }
    x.bs[0] = xsum[chunk * 64 + 2 * lane];
    x.bs[1] = xsum[chunk * 64 + 2 * lane + 1];
}

template <int DT> struct Lane;

// ---- Q4_0: 18-byte blocks, interleaved nibbles, w = (n - 8) * d --------------
template <> struct Lane<1> {
    static constexpr int STEP_W = 2048, STEP_BYTES = 1152, UNIT_W = 32, LANE_UNITS = 2, LANE_BYTES = 36;
    using X = X64;
    static TM_HD void load_x(X& x, const float4* xs4, const float* xsum, int chunk, int lane) { load_x64(x, xs4, xsum, chunk, lane); }

    template <int P0, int XB>
    static TM_HD float block(const uint32_t* lo, const uint32_t* hi, const X& x, float d, float bsum) {
        float2 a0 = mk2(0.f, 0.f), a1 = mk2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
            const int Pa = P0 + j, Pb = P0 + j + 1;
            // byte Pa holds elements 2j (low nibble) and 2j+1 (high nibble)
            a0 = fma2(mk2(byte128(lo, Pa), byte128(hi, Pa)), x.v[XB + j], a0);
            a1 = fma2(mk2(byte128(lo, Pb), byte128(hi, Pb)), x.v[XB + j + 1], a1);
        }
        const float S = (a0.x + a0.y) + (a1.x + a1.y);
        return d * fma1(-136.f, bsum, S);
    }
    // 128 + byte P of the word array (P is a compile-time constant after unrolling)
    static TM_HD float byte128(const uint32_t* w, int P) {
        switch (P & 3) {
            case 0: return code128<0>(w[P >> 2]);
            case 1: return code128<1>(w[P >> 2]);
            case 2: return code128<2>(w[P >> 2]);
            default: return code128<3>(w[P >> 2]);
        }
    }
    // p: the lane's 36 bytes (4-byte aligned); nvalid: how many of its blocks exist (1 or 2)
    static TM_HD float dot(const uint8_t* p, const X& x, int lane, int nvalid) {
        (void)lane;
        uint32_t w[9], lo[9], hi[9];
#pragma unroll
        for (int i = 0; i < 9; ++i) { w[i] = load4a(p + 4 * i); lo[i] = w[i] & kLo; hi[i] = (w[i] >> 4) & kLo; }
        float acc = block<2, 0>(lo, hi, x, half_to_float(w[0] & 0xffffu), x.bs[0]);
        if (nvalid > 1) acc += block<20, 16>(lo, hi, x, half_to_float(w[4] >> 16), x.bs[1]);
        return acc;
    }
};

// ---- Q8_0: 34-byte blocks, w = q * d -----------------------------------------
template <> struct Lane<0> {
    static constexpr int STEP_W = 2048, STEP_BYTES = 2176, UNIT_W = 32, LANE_UNITS = 2, LANE_BYTES = 68;
    using X = X64;
    static TM_HD void load_x(X& x, const float4* xs4, const float* xsum, int chunk, int lane) { load_x64(x, xs4, xsum, chunk, lane); }

    static TM_HD float byte32768(const uint32_t* w, int P) {
        switch (P & 3) {
            case 0: return code32768<0>(w[P >> 2]);
            case 1: return code32768<1>(w[P >> 2]);
            case 2: return code32768<2>(w[P >> 2]);
            default: return code32768<3>(w[P >> 2]);
        }
    }
    template <int P0, int XB>
    static TM_HD float block(const uint32_t* u, const X& x, float d) {
        float2 a0 = mk2(0.f, 0.f), a1 = mk2(0.f, 0.f);
        const float2 off = mk2(-32896.f, -32896.f);          // 32768 + the 128 of the sign flip
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
            a0 = fma2(add2(mk2(byte32768(u, P0 + i), byte32768(u, P0 + i + 1)), off), x.v[XB + i / 2], a0);
            a1 = fma2(add2(mk2(byte32768(u, P0 + i + 2), byte32768(u, P0 + i + 3)), off), x.v[XB + i / 2 + 1], a1);
        }
        return d * ((a0.x + a0.y) + (a1.x + a1.y));
    }
    static TM_HD float dot(const uint8_t* p, const X& x, int lane, int nvalid) {
        (void)lane;
        uint32_t w[17], u[17];
#pragma unroll
        for (int i = 0; i < 17; ++i) { w[i] = load4a(p + 4 * i); u[i] = w[i] ^ 0x80808080u; }
        float acc = block<2, 0>(u, x, half_to_float(w[0] & 0xffffu));
        if (nvalid > 1) acc += block<36, 16>(u, x, half_to_float(w[8] >> 16));
        return acc;
    }
};

// ---- Q4_1: 20-byte blocks, split nibbles, w = n * d + m -----------------------
template <> struct Lane<4> {
    static constexpr int STEP_W = 2048, STEP_BYTES = 1280, UNIT_W = 32, LANE_UNITS = 2, LANE_BYTES = 40;
    using X = X64;
    static TM_HD void load_x(X& x, const float4* xs4, const float* xsum, int chunk, int lane) { load_x64(x, xs4, xsum, chunk, lane); }

    template <int XB>
    static TM_HD float block(const uint32_t* w, const X& x, float bsum) {
        float2 a0 = mk2(0.f, 0.f), a1 = mk2(0.f, 0.f);
#pragma unroll
        for (int k = 0; k < 4; ++k) {                       // word k: bytes 4k..4k+3
            const uint32_t lo = w[1 + k] & kLo, hi = (w[1 + k] >> 4) & kLo;
            a0 = fma2(mk2(code128<0>(lo), code128<1>(lo)), x.v[XB + 2 * k], a0);
            a1 = fma2(mk2(code128<2>(lo), code128<3>(lo)), x.v[XB + 2 * k + 1], a1);
            a0 = fma2(mk2(code128<0>(hi), code128<1>(hi)), x.v[XB + 8 + 2 * k], a0);
            a1 = fma2(mk2(code128<2>(hi), code128<3>(hi)), x.v[XB + 8 + 2 * k + 1], a1);
        }
        const float S = (a0.x + a0.y) + (a1.x + a1.y);
        const float d = half_to_float(w[0] & 0xffffu), m = half_to_float(w[0] >> 16);
        return fma1(d, fma1(-128.f, bsum, S), m * bsum);
    }
    static TM_HD float dot(const uint8_t* p, const X& x, int lane, int nvalid) {
        (void)lane;
        uint32_t w[10];
#pragma unroll
        for (int i = 0; i < 10; ++i) w[i] = load4a(p + 4 * i);
        float acc = block<0>(w, x, x.bs[0]);
        if (nvalid > 1) acc += block<16>(w + 5, x, x.bs[1]);
        return acc;
    }
};

// ---------------------------------------------------------------------------
// Q5_K: 176-byte super-blocks of 256. Eight lanes share a super-block; lane i
// takes group g = i/2 (64 weights: sub-blocks 2g and 2g+1) and byte half q = i%2:
// bytes 16q..16q+15 of the group's qs, i.e. 16 weights of each sub-block.
// ---------------------------------------------------------------------------
template <> struct Lane<5> {
    static constexpr int STEP_W = 1024, STEP_BYTES = 704, UNIT_W = 256, LANE_UNITS = 1, LANE_BYTES = 0;
    struct X {
        float2 v[16];   // [0..7] run of sub-block 2g, [8..15] run of sub-block 2g+1
        float s0, s1;   // sums of the two runs
    };
    static TM_HD void load_x(X& x, const float4* xs4, const float* xsum, int chunk, int lane) {
        (void)xsum;
        const uint32_t S = (uint32_t)chunk * 4u + (uint32_t)(lane >> 3);
        const uint32_t g = (uint32_t)(lane & 7) >> 1, q = (uint32_t)lane & 1u;
        const uint32_t q0 = 64u * S + 16u * g + 4u * q;
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float4 a = xs4[x_slot(q0 + e)];
            const float4 b = xs4[x_slot(q0 + 8 + e)];
            x.v[2 * e] = mk2(a.x, a.y); x.v[2 * e + 1] = mk2(a.z, a.w);
            x.v[8 + 2 * e] = mk2(b.x, b.y); x.v[8 + 2 * e + 1] = mk2(b.z, b.w);
            s0 += (a.x + a.y) + (a.z + a.w);
            s1 += (b.x + b.y) + (b.z + b.w);
        }
        x.s0 = s0; x.s1 = s1;
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
        float2 a0 = mk2(0.f, 0.f), a1 = mk2(0.f, 0.f);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t t = wh[e] >> (2u * g);
            const uint32_t c0 = (wq[e] & kLo) | ((t << 4) & 0x10101010u);
            const uint32_t c1 = ((wq[e] >> 4) & kLo) | ((t << 3) & 0x10101010u);
            a0 = fma2(mk2(code128<0>(c0), code128<1>(c0)), x.v[2 * e], a0);
            a0 = fma2(mk2(code128<2>(c0), code128<3>(c0)), x.v[2 * e + 1], a0);
            a1 = fma2(mk2(code128<0>(c1), code128<1>(c1)), x.v[8 + 2 * e], a1);
            a1 = fma2(mk2(code128<2>(c1), code128<3>(c1)), x.v[8 + 2 * e + 1], a1);
        }
        const float S0 = fma1(-128.f, x.s0, a0.x + a0.y);
        const float S1 = fma1(-128.f, x.s1, a1.x + a1.y);
        const float d = half_to_float(hdr.x & 0xffffu), dmin = half_to_float(hdr.x >> 16);
        const float pos = fma1(sc[0], S0, sc[1] * S1);
        const float neg = fma1(mn[0], x.s0, mn[1] * x.s1);
        return fma1(d, pos, -(dmin * neg));
    }
};

// ---------------------------------------------------------------------------
// Q6_K: 210-byte super-blocks of 256, only 2-byte aligned. Four lanes share a
// super-block; lane i takes l in [8i, 8i+8) of both 128-halves: for each half
// 8 bytes of ql[l], 8 of ql[l+32], 8 of qh[l] -> 4 runs of 8 weights (elements
// l + 32j), each run inside one 16-weight sub-block with its own int8 scale.
// ---------------------------------------------------------------------------
template <> struct Lane<6> {
    static constexpr int STEP_W = 2048, STEP_BYTES = 1680, UNIT_W = 256, LANE_UNITS = 1, LANE_BYTES = 0;
    struct X {
        float2 v[32];   // run (h, j) at v[4*(4h+j) .. +3]
        float s8[8];    // sum of each run
    };
    static TM_HD void load_x(X& x, const float4* xs4, const float* xsum, int chunk, int lane) {
        (void)xsum;
        const uint32_t S = (uint32_t)chunk * 8u + (uint32_t)(lane >> 2);
        const uint32_t i = (uint32_t)lane & 3u;
#pragma unroll
        for (int r = 0; r < 8; ++r) {                       // r = 4h + j
            const uint32_t q0 = 64u * S + 8u * (uint32_t)r + 2u * i;
            const float4 a = xs4[x_slot(q0)];
            const float4 b = xs4[x_slot(q0 + 1)];
            x.v[4 * r] = mk2(a.x, a.y); x.v[4 * r + 1] = mk2(a.z, a.w);
            x.v[4 * r + 2] = mk2(b.x, b.y); x.v[4 * r + 3] = mk2(b.z, b.w);
            x.s8[r] = ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
        }
    }
    static TM_HD float run(uint32_t c0, uint32_t c1, const X& x, int r) {
        float2 a = mk2(0.f, 0.f);
        a = fma2(mk2(code128<0>(c0), code128<1>(c0)), x.v[4 * r], a);
        a = fma2(mk2(code128<2>(c0), code128<3>(c0)), x.v[4 * r + 1], a);
        a = fma2(mk2(code128<0>(c1), code128<1>(c1)), x.v[4 * r + 2], a);
        a = fma2(mk2(code128<2>(c1), code128<3>(c1)), x.v[4 * r + 3], a);
        return fma1(-160.f, x.s8[r], a.x + a.y);            // 128 offset + zero point 32
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
            acc = fma1((float)sc[0], run(c00, c01, x, 4 * h + 0), acc);
            acc = fma1((float)sc[2], run(c10, c11, x, 4 * h + 1), acc);
            acc = fma1((float)sc[4], run(c20, c21, x, 4 * h + 2), acc);
            acc = fma1((float)sc[6], run(c30, c31, x, 4 * h + 3), acc);
        }
        const uint32_t dh = (uint32_t)B[208] | ((uint32_t)B[209] << 8);
        return half_to_float(dh) * acc;
    }
};

}  // namespace tmc
