// qdecode.cuh — bit-exact scalar decode of one weight from a serialized block.
//
// decode_weight<DT>(row, k) returns weight k of a row exactly as the reference's
// scalar dequantizers produce it (tensormark/quant.h:194-200 Q8_0, 397-408 Q4_0,
// 267-277 Q4_1, 282-301 Q4_K, 304-330 Q5_K, 338-365 Q6_K; llama.h:4588-4597 GGUF Q4_0): the same fp32 operations in the
// same order, each rounded separately (__fmul_rn/__fadd_rn/__fsub_rn keep the
// compiler from contracting them into FMAs), and the same half->float rule for
// every encoding including subnormals and NaN payloads (quant.h:58-70).
// Used where exactness matters more than speed: the dequant kernels and the
// embedding-row gather. Byte loads only, so any address alignment works.
#pragma once

#include <stdint.h>

namespace tmc {

__device__ __forceinline__ float half_bits_exact(uint32_t h) {
    const uint32_t s = (h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 1023u;
    if (e == 31u) return __uint_as_float(s | 0x7f800000u | (m << 13));
    if (e != 0u) return __uint_as_float(s | ((e + 112u) << 23) | (m << 13));
    if (m == 0u) return __uint_as_float(s);
    return __uint_as_float(s | __float_as_uint(__fmul_rn(__uint2float_rn(m), 0x1p-24f)));
}
__device__ __forceinline__ float rd_half(const uint8_t* p) { return half_bits_exact((uint32_t)p[0] | ((uint32_t)p[1] << 8)); }

template <int DT> __device__ __forceinline__ float decode_weight(const uint8_t* row, uint32_t k);

template <> __device__ __forceinline__ float decode_weight<0>(const uint8_t* row, uint32_t k) {
    const uint8_t* b = row + (size_t)(k >> 5) * 34;
    return __fmul_rn(__int2float_rn((int)(int8_t)b[2 + (k & 31)]), rd_half(b));
}
template <> __device__ __forceinline__ float decode_weight<1>(const uint8_t* row, uint32_t k) {
    const uint8_t* b = row + (size_t)(k >> 5) * 18;
    const uint32_t e = k & 31, byte = b[2 + (e >> 1)];
    const int n = (int)((e & 1) ? (byte >> 4) : (byte & 15u)) - 8;
    return __fmul_rn(__int2float_rn(n), rd_half(b));
}
template <> __device__ __forceinline__ float decode_weight<9>(const uint8_t* row, uint32_t k) {   // GGUF Q4_0, llama.h:4588-4597
    const uint8_t* b = row + (size_t)(k >> 5) * 18;
    const uint32_t e = k & 31, byte = b[2 + (e & 15)];
    const int n = (int)((e & 16) ? (byte >> 4) : (byte & 15u)) - 8;
    return __fmul_rn(rd_half(b), __int2float_rn(n));
}
template <> __device__ __forceinline__ float decode_weight<7>(const uint8_t* row, uint32_t k) {   // TQ2, quant.h:507-515
    const uint8_t* b = row + (size_t)(k >> 7) * 34;
    const uint32_t e = k & 127;
    const int code = (int)((b[2 + (e >> 2)] >> (2 * (e & 3))) & 3u) - 1;
    return __fmul_rn(__int2float_rn(code), rd_half(b));
}
template <> __device__ __forceinline__ float decode_weight<4>(const uint8_t* row, uint32_t k) {
    const uint8_t* b = row + (size_t)(k >> 5) * 20;
    const uint32_t e = k & 31, byte = b[4 + (e & 15)];
    const uint32_t n = (e & 16) ? (byte >> 4) : (byte & 15u);
    return __fadd_rn(__fmul_rn(__uint2float_rn(n), rd_half(b)), rd_half(b + 2));
}
template <> __device__ __forceinline__ float decode_weight<5>(const uint8_t* row, uint32_t k) {
    const uint8_t* b = row + (size_t)(k >> 8) * 176;
    const uint32_t e = k & 255, j = e >> 5, g = j >> 1, l = e & 31;
    const uint8_t* sc = b + 4;
    uint32_t s6, m6;
    if (j < 4) { s6 = sc[j] & 63u; m6 = sc[j + 4] & 63u; }
    else { s6 = (sc[j + 4] & 15u) | ((uint32_t)(sc[j - 4] >> 6) << 4); m6 = (uint32_t)(sc[j + 4] >> 4) | ((uint32_t)(sc[j] >> 6) << 4); }
    const uint32_t byte = b[48 + 32 * g + l];
    const uint32_t code = ((j & 1) ? (byte >> 4) : (byte & 15u)) + (((b[16 + l] >> j) & 1u) << 4);
    const float d1 = __fmul_rn(rd_half(b), __uint2float_rn(s6));
    const float m1 = __fmul_rn(rd_half(b + 2), __uint2float_rn(m6));
    return __fsub_rn(__fmul_rn(d1, __uint2float_rn(code)), m1);
}
template <> __device__ __forceinline__ float decode_weight<8>(const uint8_t* row, uint32_t k) {   // Q4_K, quant.h:282-301
    const uint8_t* b = row + (size_t)(k >> 8) * 144;
    const uint32_t e = k & 255, j = e >> 5, g = j >> 1, l = e & 31;
    const uint8_t* sc = b + 4;
    uint32_t s6, m6;
    if (j < 4) { s6 = sc[j] & 63u; m6 = sc[j + 4] & 63u; }
    else { s6 = (sc[j + 4] & 15u) | ((uint32_t)(sc[j - 4] >> 6) << 4); m6 = (uint32_t)(sc[j + 4] >> 4) | ((uint32_t)(sc[j] >> 6) << 4); }
    const uint32_t byte = b[16 + 32 * g + l];
    const uint32_t code = (j & 1) ? (byte >> 4) : (byte & 15u);
    const float d1 = __fmul_rn(rd_half(b), __uint2float_rn(s6));
    const float m1 = __fmul_rn(rd_half(b + 2), __uint2float_rn(m6));
    return __fsub_rn(__fmul_rn(d1, __uint2float_rn(code)), m1);
}
template <> __device__ __forceinline__ float decode_weight<6>(const uint8_t* row, uint32_t k) {
    const uint8_t* b = row + (size_t)(k >> 8) * 210;
    const uint32_t e = k & 255, h = e >> 7, j = (e >> 5) & 3, l = e & 31;
    const uint32_t qlb = b[64 * h + 32 * (j & 1) + l];
    const uint32_t lo = (j & 2) ? (qlb >> 4) : (qlb & 15u);
    const uint32_t hi = (b[128 + 32 * h + l] >> (2 * j)) & 3u;
    const int code = (int)(lo | (hi << 4)) - 32;
    const float ds = __fmul_rn(rd_half(b + 208), __int2float_rn((int)(int8_t)b[192 + 8 * h + 2 * j + (l >> 4)]));
    return __fmul_rn(ds, __int2float_rn(code));
}

// Runtime-dtype form for the few callers that are not templated.
__device__ __forceinline__ float decode_weight_dt(unsigned dt, const uint8_t* row, uint32_t k) {
    switch (dt) {
        case 0: return decode_weight<0>(row, k);
        case 1: return decode_weight<1>(row, k);
        case 4: return decode_weight<4>(row, k);
        case 5: return decode_weight<5>(row, k);
        case 7: return decode_weight<7>(row, k);
        case 8: return decode_weight<8>(row, k);
        case 9: return decode_weight<9>(row, k);
        default: return decode_weight<6>(row, k);
    }
}

}  // namespace tmc
