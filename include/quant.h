// include/quant.h — serialized block formats of the quantized-weight matmul path.
//
// Host-side mirror of the reference's block structs and scalar dequantizers
// (tensormark/quant.h:35-49 Q8_0/Q4_0, 214-249 Q4_1/Q5_K/Q6_K, 256-264 the
// 6-bit scale/min unpack, 194-200 / 267-277 / 304-330 / 338-365 / 397-408 the
// dequantizers, 58-87 and 120-146 the fp16 conversions). Names, namespace and
// byte layouts are the reference's so a caller of its header compiles against
// this one; the bodies are written for this project. The arithmetic order of
// every dequantizer is part of the contract (the CUDA dequant kernels are
// bit-exact against it), so each multiply/add below is a separate fp32
// operation: build host code that includes this header with -ffp-contract=off.
//
// dtype ids (tensormark/tmq.h:48-60): 0 Q8_0, 1 Q4_0, 3 F16, 4 Q4_1, 5 Q5_K,
// 6 Q6_K, 8 Q4_K. Geometry (tmq.h:83-115): block_elems / block_bytes below.
#pragma once

#include <bit>
#include <cstddef>
#include <cstdint>
#include <stdexcept>

namespace tmq {

constexpr int kBlock = 32;     // weights per Q8_0/Q4_0/Q4_1 block
constexpr int kKBlock = 256;   // weights per K-quant super-block

#pragma pack(push, 1)
struct BlockQ8_0 {             // w = q * d
    std::uint16_t d_fp16;
    std::int8_t   qs[32];
};
struct BlockQ4_0 {             // w = (nibble - 8) * d; byte j: low = elem 2j, high = elem 2j+1
    std::uint16_t d_fp16;
    std::uint8_t  qs[16];
};
struct BlockQ4_1 {             // w = nibble * d + m; byte j: low = elem j, high = elem j+16
    std::uint16_t d_fp16;
    std::uint16_t m_fp16;
    std::uint8_t  qs[16];
};
struct BlockQ4_K {             // w = (d*sc)*nibble - (dmin*mn); dtype 8 (tmq.h:57)
    std::uint16_t d_fp16;
    std::uint16_t dmin_fp16;
    std::uint8_t  scales[12];  // 8 (scale, min) pairs, 6 bits each
    std::uint8_t  qs[128];     // byte 32g+l: low = elem 64g+l, high = elem 64g+32+l
};
struct BlockQ5_K {             // w = (d*sc)*code - (dmin*mn), code = nibble + 16*hibit
    std::uint16_t d_fp16;
    std::uint16_t dmin_fp16;
    std::uint8_t  scales[12];  // 8 (scale, min) pairs, 6 bits each
    std::uint8_t  qh[32];      // bit 2g / 2g+1 of byte l: high bit of elem 64g+l / 64g+32+l
    std::uint8_t  qs[128];     // byte 32g+l: low = elem 64g+l, high = elem 64g+32+l
};
struct BlockQ6_K {             // w = (d*sc[sub])*(code-32)
    std::uint8_t  ql[128];
    std::uint8_t  qh[64];
    std::int8_t   scales[16];
    std::uint16_t d_fp16;      // last, byte offset 208
};
#pragma pack(pop)

static_assert(sizeof(BlockQ8_0) == 34 && alignof(BlockQ8_0) == 1);
static_assert(sizeof(BlockQ4_0) == 18 && alignof(BlockQ4_0) == 1);
static_assert(sizeof(BlockQ4_1) == 20 && alignof(BlockQ4_1) == 1);
static_assert(sizeof(BlockQ4_K) == 144 && alignof(BlockQ4_K) == 1);
static_assert(sizeof(BlockQ5_K) == 176 && alignof(BlockQ5_K) == 1);
static_assert(sizeof(BlockQ6_K) == 210 && alignof(BlockQ6_K) == 1);

enum class Dtype : std::uint32_t { Q8_0 = 0, Q4_0 = 1, F32 = 2, F16 = 3, Q4_1 = 4, Q5_K = 5, Q6_K = 6, TQ2 = 7, Q4_K = 8, GGUF_Q4_0 = 9, BF16 = 10 };

constexpr std::uint32_t block_elems(std::uint32_t dtype) {
    switch (dtype) {
        case 0: case 1: case 4: case 9: return 32;
        case 5: case 6: case 8: return 256;
        case 7: return 128;
        case 2: case 3: case 10: return 1;
        default: return 0;
    }
}
constexpr std::size_t block_bytes(std::uint32_t dtype) {
    switch (dtype) {
        case 0: case 7: return 34; case 1: case 9: return 18; case 2: return 4; case 3: case 10: return 2;
        case 4: return 20; case 5: return 176; case 6: return 210; case 8: return 144;
        default: return 0;
    }
}
// Payload bytes of an out x in tensor; 0 when `in` is not whole blocks.
constexpr std::size_t weight_bytes(std::uint32_t dtype, std::size_t out, std::size_t in) {
    const std::size_t e = block_elems(dtype);
    return (e == 0 || in % e != 0) ? 0 : out * (in / e) * block_bytes(dtype);
}

// ---- IEEE half <-> float -------------------------------------------------
// Exact for every encoding: subnormals are man * 2^-24, NaN payloads are kept
// in the top mantissa bits (reference quant.h:58-70).
inline float fp16_to_fp32(std::uint16_t h) {
    const std::uint32_t s = (std::uint32_t)(h >> 15) << 31;
    const std::uint32_t e = (h >> 10) & 31u;
    const std::uint32_t f = h & 1023u;
    std::uint32_t bits;
    if (e == 31u) {
        bits = s | 0x7f800000u | (f << 13);
    } else if (e != 0u) {
        bits = s | ((e + 112u) << 23) | (f << 13);
    } else if (f == 0u) {
        bits = s;
    } else {
        const float mag = (float)f * 0x1p-24f;
        bits = s | std::bit_cast<std::uint32_t>(mag);
    }
    return std::bit_cast<float>(bits);
}

// Round-to-nearest-even float -> half; overflow to infinity, underflow through
// the subnormal range to signed zero (reference quant.h:120-146).
inline std::uint16_t fp32_to_fp16(float v) {
    const std::uint32_t u = std::bit_cast<std::uint32_t>(v);
    const std::uint32_t s = (u >> 16) & 0x8000u;
    const std::uint32_t e8 = (u >> 23) & 255u;
    const std::uint32_t frac = u & 0x7fffffu;
    if (e8 == 255u) return (std::uint16_t)(s | 0x7c00u | (frac ? 0x200u : 0u));
    const int e = (int)e8 - 112;                 // half exponent field
    if (e >= 31) return (std::uint16_t)(s | 0x7c00u);
    auto round_shift = [](std::uint32_t m, int sh) {
        const std::uint32_t keep = m >> sh;
        const std::uint32_t lost = m & ((1u << sh) - 1u);
        const std::uint32_t half = 1u << (sh - 1);
        return keep + ((lost > half || (lost == half && (keep & 1u))) ? 1u : 0u);
    };
    if (e <= 0) {
        if (e < -10) return (std::uint16_t)s;
        return (std::uint16_t)(s | round_shift(frac | 0x800000u, 14 - e));
    }
    // A mantissa carry out of the rounding walks into the exponent field, which
    // is exactly the next binade (and infinity from the top one).
    return (std::uint16_t)(s | (((std::uint32_t)e << 10) + round_shift(frac, 13)));
}

// 6-bit (scale, min) pair j of a Q5_K `scales` array (reference quant.h:256-264).
inline void k_scale_min(int j, const std::uint8_t* q, std::uint8_t& d, std::uint8_t& m) {
    if (j < 4) {
        d = q[j] & 63u;
        m = q[j + 4] & 63u;
    } else {
        d = (std::uint8_t)((q[j + 4] & 15u) | ((q[j - 4] >> 6) << 4));
        m = (std::uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

namespace detail {
inline void need_rows(const void* in, const void* out, std::size_t n, std::size_t per) {
    if (n % per != 0 || (n != 0 && (!in || !out)))
        throw std::invalid_argument("quantized rows require complete blocks and non-null buffers");
}
}  // namespace detail

inline void dequantize_row_q8_0(const BlockQ8_0* in, float* x, std::size_t n) {
    detail::need_rows(in, x, n, kBlock);
    for (std::size_t b = 0; b < n / kBlock; ++b) {
        const float d = fp16_to_fp32(in[b].d_fp16);
        for (int i = 0; i < kBlock; ++i) x[b * kBlock + i] = (float)in[b].qs[i] * d;
    }
}

inline void dequantize_row_q4_0(const BlockQ4_0* in, float* x, std::size_t n) {
    detail::need_rows(in, x, n, kBlock);
    for (std::size_t b = 0; b < n / kBlock; ++b) {
        const float d = fp16_to_fp32(in[b].d_fp16);
        for (int j = 0; j < 16; ++j) {
            const int byte = in[b].qs[j];
            x[b * kBlock + 2 * j]     = (float)((byte & 15) - 8) * d;
            x[b * kBlock + 2 * j + 1] = (float)((byte >> 4) - 8) * d;
        }
    }
}

inline void dequantize_row_q4_1(const BlockQ4_1* in, float* x, std::size_t n) {
    detail::need_rows(in, x, n, kBlock);
    for (std::size_t b = 0; b < n / kBlock; ++b) {
        const float d = fp16_to_fp32(in[b].d_fp16);
        const float m = fp16_to_fp32(in[b].m_fp16);
        for (int j = 0; j < 16; ++j) {
            const float lo = (float)(in[b].qs[j] & 15u) * d;
            const float hi = (float)(in[b].qs[j] >> 4) * d;
            x[b * kBlock + j]      = lo + m;
            x[b * kBlock + j + 16] = hi + m;
        }
    }
}

// reference quant.h:282-301
inline void dequantize_row_q4_K(const BlockQ4_K* in, float* x, std::size_t n) {
    detail::need_rows(in, x, n, kKBlock);
    for (std::size_t b = 0; b < n / kKBlock; ++b) {
        const BlockQ4_K& k = in[b];
        float* y = x + b * kKBlock;
        const float d = fp16_to_fp32(k.d_fp16);
        const float dmin = fp16_to_fp32(k.dmin_fp16);
        for (int g = 0; g < 4; ++g) {
            for (int half = 0; half < 2; ++half) {
                std::uint8_t sc, mn;
                k_scale_min(2 * g + half, k.scales, sc, mn);
                const float dl = d * (float)sc;
                const float ml = dmin * (float)mn;
                for (int l = 0; l < 32; ++l) {
                    const int nib = half ? (k.qs[32 * g + l] >> 4) : (k.qs[32 * g + l] & 15);
                    const float prod = dl * (float)nib;
                    y[64 * g + 32 * half + l] = prod - ml;
                }
            }
        }
    }
}

inline void dequantize_row_q5_K(const BlockQ5_K* in, float* x, std::size_t n) {
    detail::need_rows(in, x, n, kKBlock);
    for (std::size_t b = 0; b < n / kKBlock; ++b) {
        const BlockQ5_K& k = in[b];
        float* y = x + b * kKBlock;
        const float d = fp16_to_fp32(k.d_fp16);
        const float dmin = fp16_to_fp32(k.dmin_fp16);
        for (int g = 0; g < 4; ++g) {              // 64 weights per group: two 32-sub-blocks
            for (int half = 0; half < 2; ++half) {
                std::uint8_t sc, mn;
                k_scale_min(2 * g + half, k.scales, sc, mn);
                const float dl = d * (float)sc;
                const float ml = dmin * (float)mn;
                const int hbit = 1 << (2 * g + half);
                for (int l = 0; l < 32; ++l) {
                    const int nib = half ? (k.qs[32 * g + l] >> 4) : (k.qs[32 * g + l] & 15);
                    const int code = nib + ((k.qh[l] & hbit) ? 16 : 0);
                    const float prod = dl * (float)code;
                    y[64 * g + 32 * half + l] = prod - ml;
                }
            }
        }
    }
}

inline void dequantize_row_q6_K(const BlockQ6_K* in, float* x, std::size_t n) {
    detail::need_rows(in, x, n, kKBlock);
    for (std::size_t b = 0; b < n / kKBlock; ++b) {
        const BlockQ6_K& k = in[b];
        const float d = fp16_to_fp32(k.d_fp16);
        for (int h = 0; h < 2; ++h) {              // two halves of 128 weights
            const std::uint8_t* ql = k.ql + 64 * h;
            const std::uint8_t* qh = k.qh + 32 * h;
            const std::int8_t*  sc = k.scales + 8 * h;
            float* y = x + b * kKBlock + 128 * h;
            for (int j = 0; j < 4; ++j) {          // element l + 32j
                for (int l = 0; l < 32; ++l) {
                    const int lo = (j & 2) ? (ql[l + 32 * (j & 1)] >> 4) : (ql[l + 32 * (j & 1)] & 15);
                    const int hi = (qh[l] >> (2 * j)) & 3;
                    const int code = (lo | (hi << 4)) - 32;
                    const float ds = d * (float)sc[l / 16 + 2 * j];
                    y[l + 32 * j] = ds * (float)code;
                }
            }
        }
    }
}

// TQ2 (container dtype 7): 34-byte blocks of 128 ternary-coded weights, four 2-bit codes per byte, low bits first,
// w = (code - 1) * d (tensormark/quant.h:452-456, 507-515).
struct BlockTq2_34x128 {
    std::uint16_t d_fp16;
    std::uint8_t qs[32];
} __attribute__((packed));
static_assert(sizeof(BlockTq2_34x128) == 34 && alignof(BlockTq2_34x128) == 1);
inline void dequantize_row_tq2_34x128(const BlockTq2_34x128* in, float* x, std::size_t n) {
    detail::need_rows(in, x, n, 128);
    for (std::size_t b = 0; b < n / 128; ++b, x += 128) {
        const float d = fp16_to_fp32(in[b].d_fp16);
        for (int j = 0; j < 128; ++j) x[j] = static_cast<float>(static_cast<int>((in[b].qs[j >> 2] >> (2 * (j & 3))) & 3u) - 1) * d;
    }
}

// GGUF's own Q4_0 (container dtype 9): split nibbles, byte j = elements j | j + 16 (tensormark/llama.h:4588-4597).
inline void dequantize_row_gguf_q4_0(const BlockQ4_0* in, float* x, std::size_t n) {
    detail::need_rows(in, x, n, kBlock);
    for (std::size_t b = 0; b < n / kBlock; ++b, x += kBlock) {
        const float d = fp16_to_fp32(in[b].d_fp16);
        for (int j = 0; j < 16; ++j) {
            x[j] = d * static_cast<float>((in[b].qs[j] & 15) - 8);
            x[j + 16] = d * static_cast<float>((in[b].qs[j] >> 4) - 8);
        }
    }
}
// A split-nibble block rewritten as the container's interleaved Q4_0 block: same scale, same 32 codes, so the weights
// are bit-identical (what tensormark/convert_gguf.cpp:124-135 does when it converts a GGUF file). src may equal dst.
inline void q4_split_to_interleaved(const BlockQ4_0* src, BlockQ4_0* dst, std::size_t nblocks) {
    for (std::size_t b = 0; b < nblocks; ++b) {
        std::uint8_t code[32];
        for (int j = 0; j < 16; ++j) { code[j] = src[b].qs[j] & 15; code[j + 16] = static_cast<std::uint8_t>(src[b].qs[j] >> 4); }
        dst[b].d_fp16 = src[b].d_fp16;
        for (int j = 0; j < 16; ++j) dst[b].qs[j] = static_cast<std::uint8_t>(code[2 * j] | (code[2 * j + 1] << 4));
    }
}

// Dequantize `n` weights of any block dtype served by the matmul path.
inline void dequantize_row(std::uint32_t dtype, const void* in, float* x, std::size_t n) {
    switch (dtype) {
        case 0: dequantize_row_q8_0(static_cast<const BlockQ8_0*>(in), x, n); break;
        case 1: dequantize_row_q4_0(static_cast<const BlockQ4_0*>(in), x, n); break;
        case 4: dequantize_row_q4_1(static_cast<const BlockQ4_1*>(in), x, n); break;
        case 5: dequantize_row_q5_K(static_cast<const BlockQ5_K*>(in), x, n); break;
        case 6: dequantize_row_q6_K(static_cast<const BlockQ6_K*>(in), x, n); break;
        case 7: dequantize_row_tq2_34x128(static_cast<const BlockTq2_34x128*>(in), x, n); break;
        case 8: dequantize_row_q4_K(static_cast<const BlockQ4_K*>(in), x, n); break;
        case 9: dequantize_row_gguf_q4_0(static_cast<const BlockQ4_0*>(in), x, n); break;
        default: throw std::invalid_argument("dequantize_row: dtype is not a block format");
    }
}

}  // namespace tmq
