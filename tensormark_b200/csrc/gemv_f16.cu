// gemv_f16.cu — y = W x for tensors that a container keeps as plain 16-bit rows (fp16, dtype 3; bf16, dtype 10), the
// embedding-row gather from such a table, and the in-place nibble reorder that turns GGUF's Q4_0 blocks into the
// container's.
//
// Replaces the reference's f16_gemv_coop_r1/2/4 (tensormark/metal.h:575-613, host side tok_gemv_h 3693-3721) and
// embed_h_row (2396-2407, tok_embed_h 3260-3271); bf16 has no GPU kernel in the reference (its loader keeps such
// tensors on the CPU, tensormark/llama.h:4599-4606) and is served by the same kernel here.
//
// Bound: HBM, 2 bytes per weight. x is copied into shared memory once per CTA as fp32; a warp owns a row at a time and
// its lanes read the row as 16-byte pieces (eight weights), four independent loads in flight per lane, fp32 FMA, one
// shuffle reduction per row. Rows must be 16-byte aligned for that form (K a multiple of 8 and an aligned base);
// anything else takes a scalar-load kernel with the same arithmetic.
#include "common.cuh"

#include <cuda_fp16.h>

namespace tmc {
namespace {

template <bool BF16> __device__ __forceinline__ float2 pair_to_float(uint32_t u) {
    if constexpr (BF16) return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
    else return __half22float2(*reinterpret_cast<const __half2*>(&u));
}
template <bool BF16> __device__ __forceinline__ float one_to_float(uint16_t h) {
    if constexpr (BF16) return __uint_as_float((uint32_t)h << 16);
    else return __half2float(__ushort_as_half(h));
}
__device__ __forceinline__ float warp_total(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
template <bool BF16> __device__ __forceinline__ float dot8(const uint4 w, const float* xs) {
    const float4 a = *reinterpret_cast<const float4*>(xs), b = *reinterpret_cast<const float4*>(xs + 4);
    const float2 p0 = pair_to_float<BF16>(w.x), p1 = pair_to_float<BF16>(w.y), p2 = pair_to_float<BF16>(w.z), p3 = pair_to_float<BF16>(w.w);
    float s = p0.x * a.x;
    s = fmaf(p0.y, a.y, s); s = fmaf(p1.x, a.z, s); s = fmaf(p1.y, a.w, s);
    s = fmaf(p2.x, b.x, s); s = fmaf(p2.y, b.y, s); s = fmaf(p3.x, b.z, s); s = fmaf(p3.y, b.w, s);
    return s;
}

template <bool BF16>
__global__ void __launch_bounds__(256) gemv_half_rows(const float* __restrict__ x, const uint16_t* __restrict__ W, float* __restrict__ y,
                                                      uint32_t N, uint32_t K) {
    extern __shared__ __align__(16) float xs[];
    asm volatile("griddepcontrol.wait;" ::: "memory");          // x may come from the preceding kernel of the stream
    for (uint32_t i = threadIdx.x; i < K / 4; i += blockDim.x) reinterpret_cast<float4*>(xs)[i] = __ldcg(reinterpret_cast<const float4*>(x) + i);
    __syncthreads();
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, k8 = K / 8;
    for (uint32_t row = blockIdx.x * 8 + warp; row < N; row += gridDim.x * 8) {
        const uint4* wr = reinterpret_cast<const uint4*>(W + (size_t)row * K);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t i = lane;
        for (; i + 96 < k8; i += 128) {                         // four 16-byte loads in flight per lane
            const uint4 w0 = __ldg(wr + i), w1 = __ldg(wr + i + 32), w2 = __ldg(wr + i + 64), w3 = __ldg(wr + i + 96);
            acc[0] += dot8<BF16>(w0, xs + 8 * i); acc[1] += dot8<BF16>(w1, xs + 8 * (i + 32));
            acc[2] += dot8<BF16>(w2, xs + 8 * (i + 64)); acc[3] += dot8<BF16>(w3, xs + 8 * (i + 96));
        }
        for (; i < k8; i += 32) acc[0] += dot8<BF16>(__ldg(wr + i), xs + 8 * i);
        const float v = warp_total((acc[0] + acc[1]) + (acc[2] + acc[3]));
        if (lane == 0) y[row] = v;
    }
}

// any K, any 2-byte aligned base: one warp per row, scalar loads
template <bool BF16>
__global__ void __launch_bounds__(256) gemv_half_generic(const float* __restrict__ x, const uint16_t* __restrict__ W, float* __restrict__ y,
                                                         uint32_t N, uint32_t K) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, row = blockIdx.x * 8 + warp;
    if (row >= N) return;
    const uint16_t* wr = W + (size_t)row * K;
    float acc = 0.f;
    for (uint32_t k = lane; k < K; k += 32) acc = fmaf(one_to_float<BF16>(wr[k]), __ldcg(x + k), acc);
    acc = warp_total(acc);
    if (lane == 0) y[row] = acc;
}

// x = row tok[idx] of a 16-bit table (sentinel 0xFFFFFFFF -> zeros), embed_h_row (metal.h:2396-2407)
template <bool BF16>
__global__ void embed_half_row(const uint32_t* __restrict__ tok, uint32_t idx, const uint16_t* __restrict__ W, float* __restrict__ x, uint32_t D) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= D) return;
    const uint32_t row = tok[idx];
    x[k] = row == 0xFFFFFFFFu ? 0.f : one_to_float<BF16>(W[(size_t)row * D + k]);
}

// GGUF Q4_0 (split nibbles: byte j = elements j | j + 16) -> container Q4_0 (byte j = elements 2j | 2j + 1), in place,
// one thread per 18-byte block (tensormark/convert_gguf.cpp:124-135). Scale and codes are unchanged, so the weights are
// bit-identical.
__global__ void q4_split_to_interleaved_kernel(uint8_t* blocks, size_t nblocks) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    uint8_t* q = blocks + b * 18 + 2;
    uint8_t s[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) s[j] = q[j];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        q[j] = (uint8_t)((s[2 * j] & 15) | ((s[2 * j + 1] & 15) << 4));
        q[j + 8] = (uint8_t)((s[2 * j] >> 4) | ((s[2 * j + 1] >> 4) << 4));
    }
}

}  // namespace

bool launch_gemv_half(const float* x, const void* W, float* y, unsigned N, unsigned K, bool bf16, cudaStream_t st) {
    if (!x || !W || !y) return fail("gemv_h: null pointer");
    if (N == 0) return true;
    if (K == 0) return fail("gemv_h: empty rows");
    if ((uintptr_t)W % 2 || (uintptr_t)x % 4) return fail("gemv_h: misaligned operand");
    const uint16_t* w = (const uint16_t*)W;
    const size_t smem = (size_t)K * 4;
    if (K % 8 == 0 && (uintptr_t)W % 16 == 0 && (uintptr_t)x % 16 == 0 && smem <= 200 * 1024) {
        unsigned grid = (N + 7) / 8;
        const unsigned cap = (unsigned)device_sm_count() * 4;
        if (grid > cap) grid = cap;
        static bool attr[2] = {false, false};
        if (smem > 48 * 1024 && !attr[bf16]) {
            const cudaError_t e = bf16 ? cudaFuncSetAttribute(gemv_half_rows<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
                                       : cudaFuncSetAttribute(gemv_half_rows<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return fail("gemv_h: cannot raise the dynamic shared memory limit");
            attr[bf16] = true;
        }
        if (bf16) gemv_half_rows<true><<<grid, 256, smem, st>>>(x, w, y, N, K);
        else gemv_half_rows<false><<<grid, 256, smem, st>>>(x, w, y, N, K);
    } else {
        if (bf16) gemv_half_generic<true><<<(N + 7) / 8, 256, 0, st>>>(x, w, y, N, K);
        else gemv_half_generic<false><<<(N + 7) / 8, 256, 0, st>>>(x, w, y, N, K);
    }
    note_launch();
    return check_launch("gemv_h");
}

bool launch_embed_half(const unsigned* tok, unsigned idx, const void* W, float* x, unsigned D, bool bf16, cudaStream_t st) {
    if (!tok || !W || !x || D == 0) return fail("embed_h: bad arguments");
    if (bf16) embed_half_row<true><<<(D + 255) / 256, 256, 0, st>>>(tok, idx, (const uint16_t*)W, x, D);
    else embed_half_row<false><<<(D + 255) / 256, 256, 0, st>>>(tok, idx, (const uint16_t*)W, x, D);
    note_launch();
    return check_launch("embed_h");
}

bool launch_q4_split_to_interleaved(uint8_t* blocks, size_t nblocks, cudaStream_t st) {
    if (!blocks) return fail("q4 repack: null pointer");
    if (nblocks == 0) return true;
    q4_split_to_interleaved_kernel<<<(unsigned)((nblocks + 255) / 256), 256, 0, st>>>(blocks, nblocks);
    note_launch();
    return check_launch("q4 repack");
}

}  // namespace tmc
