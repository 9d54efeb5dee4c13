// oracle/ref_wrap.cpp — C entry points over the reference's OWN quant.h.
//
// TEST INFRASTRUCTURE. This file contains no arithmetic: it includes the
// reference header where it lies (the include path is given by the Makefile)
// and forwards to tmq::dequantize_row_* and the fp16 conversions, so the
// restated oracle and the committed golden vectors can be pinned against the
// reference's code itself. Built with -ffp-contract=off, the unfused
// evaluation the bit-exact gate is defined on.
#include "quant.h"

#include <cstddef>
#include <cstdint>

extern "C" {
__attribute__((visibility("default"))) int tmref_dequant(int dtype, const void* blocks, float* out, std::size_t n) {
    try {
        switch (dtype) {
            case 0: tmq::dequantize_row_q8_0(static_cast<const tmq::BlockQ8_0*>(blocks), out, n); return 1;
            case 1: tmq::dequantize_row_q4_0(static_cast<const tmq::BlockQ4_0*>(blocks), out, n); return 1;
            case 4: tmq::dequantize_row_q4_1(static_cast<const tmq::BlockQ4_1*>(blocks), out, n); return 1;
            case 5: tmq::dequantize_row_q5_K(static_cast<const tmq::BlockQ5_K*>(blocks), out, n); return 1;
            case 6: tmq::dequantize_row_q6_K(static_cast<const tmq::BlockQ6_K*>(blocks), out, n); return 1;
            case 7: tmq::dequantize_row_tq2_34x128(static_cast<const tmq::BlockTq2_34x128*>(blocks), out, n); return 1;
            case 8: tmq::dequantize_row_q4_K(static_cast<const tmq::BlockQ4_K*>(blocks), out, n); return 1;
            default: return 0;
        }
    } catch (...) { return 0; }
}
__attribute__((visibility("default"))) float tmref_fp16_to_fp32(std::uint16_t h) { return tmq::fp16_to_fp32(h); }
__attribute__((visibility("default"))) std::uint16_t tmref_fp32_to_fp16(float f) { return tmq::fp32_to_fp16(f); }
__attribute__((visibility("default"))) void tmref_quantize_q4_0(const float* x, void* out, std::size_t n) {
    tmq::quantize_row_q4_0(x, static_cast<tmq::BlockQ4_0*>(out), n);
}
__attribute__((visibility("default"))) void tmref_quantize_tq2(const float* x, void* out, std::size_t n) {
    tmq::quantize_row_tq2_34x128(x, static_cast<tmq::BlockTq2_34x128*>(out), n);
}
__attribute__((visibility("default"))) void tmref_quantize_q8_0(const float* x, void* out, std::size_t n) {
    tmq::quantize_row_q8_0(x, static_cast<tmq::BlockQ8_0*>(out), n);
}
}
