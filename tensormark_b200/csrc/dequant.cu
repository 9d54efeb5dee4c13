// dequant.cu — block-quantized weights -> dense fp32 / fp16, bit-exact.
//
// fp32 output is the parity gate of the path: every value equals what
// tmq::dequantize_row_* (tensormark/quant.h:194-408) yields for the same bytes.
// It is also the fp32 form of the reference's q4_dequant_f32 (metal.h:1516-1562),
// extended to every block dtype. The fp16 output rounds that exact fp32 value
// once (round to nearest even), as q4_dequant_f16 does.
#include "common.cuh"
#include "qdecode.cuh"

#include <cuda_fp16.h>

namespace tmc {

namespace {

// One thread per 4 consecutive weights of a row; consecutive threads write
// consecutive float4s, so stores are fully coalesced. Reads are byte loads that
// hit L1 after the first touch of a block.
template <int DT, bool HALF>
__global__ void __launch_bounds__(256) dequant_rows(const uint8_t* __restrict__ W, void* __restrict__ out,
                                                     uint32_t N, uint32_t K, uint32_t row_bytes) {
    const uint64_t quad = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t total = (uint64_t)N * (K / 4);
    if (quad >= total) return;
    const uint32_t row = (uint32_t)(quad / (K / 4)), k = (uint32_t)(quad % (K / 4)) * 4;
    const uint8_t* r = W + (size_t)row * row_bytes;
    const float a = decode_weight<DT>(r, k), b = decode_weight<DT>(r, k + 1);
    const float c = decode_weight<DT>(r, k + 2), d = decode_weight<DT>(r, k + 3);
    if (HALF) {
        __half2* o = reinterpret_cast<__half2*>(out) + quad * 2;
        o[0] = __floats2half2_rn(a, b);
        o[1] = __floats2half2_rn(c, d);
    } else {
        reinterpret_cast<float4*>(out)[quad] = make_float4(a, b, c, d);
    }
}

template <bool HALF>
bool launch(const uint8_t* W, void* out, unsigned N, unsigned K, unsigned dtype, cudaStream_t st) {
    const unsigned be = block_elems(dtype);
    if (!be || dtype == DT_F16) return fail("dequant: dtype %u is not a block format", dtype);
    if (!W || !out) return fail("dequant: null pointer");
    if (N == 0) return true;
    if (K == 0 || K % be) return fail("dequant: K=%u is not a multiple of %u", K, be);
    if ((uintptr_t)out % 16) return fail("dequant: output must be 16-byte aligned");
    const uint32_t row_bytes = (K / be) * block_bytes(dtype);
    const uint64_t total = (uint64_t)N * (K / 4);
    const unsigned grid = (unsigned)((total + 255) / 256);
    switch (dtype) {
        case DT_Q8_0: dequant_rows<0, HALF><<<grid, 256, 0, st>>>(W, out, N, K, row_bytes); break;
        case DT_Q4_0: dequant_rows<1, HALF><<<grid, 256, 0, st>>>(W, out, N, K, row_bytes); break;
        case DT_Q4_1: dequant_rows<4, HALF><<<grid, 256, 0, st>>>(W, out, N, K, row_bytes); break;
        case DT_Q5_K: dequant_rows<5, HALF><<<grid, 256, 0, st>>>(W, out, N, K, row_bytes); break;
        case DT_Q4_K: dequant_rows<8, HALF><<<grid, 256, 0, st>>>(W, out, N, K, row_bytes); break;
        case DT_TQ2: dequant_rows<7, HALF><<<grid, 256, 0, st>>>(W, out, N, K, row_bytes); break;
        case DT_GGUF_Q4_0: dequant_rows<9, HALF><<<grid, 256, 0, st>>>(W, out, N, K, row_bytes); break;
        default:      dequant_rows<6, HALF><<<grid, 256, 0, st>>>(W, out, N, K, row_bytes); break;
    }
    note_launch();
    return check_launch("dequant_rows");
}

}  // namespace

bool launch_dequant(const uint8_t* W, float* out, unsigned N, unsigned K, unsigned dtype, cudaStream_t st) {
    return launch<false>(W, out, N, K, dtype, st);
}
bool launch_dequant_half(const uint8_t* W, void* out_half, unsigned N, unsigned K, unsigned dtype, cudaStream_t st) {
    return launch<true>(W, out_half, N, K, dtype, st);
}

}  // namespace tmc
