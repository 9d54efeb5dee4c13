// gemm.cu — prefill GEMM on the 5th-generation tensor cores:  C[M x N] = A[M x K] * W^T.
//
// Replaces the reference's prefill GEMMs (tensormark/metal.h:1387-1449 sgemm_q4,
// 1137-1381 q4_mm_tile*, and the dequantize + MPSMatrixMultiplication path
// 1658-1718) and covers the K-quant LM head for which the reference has no GPU
// GEMM at all (its CPU path dequantizes and calls sgemm, llama.h:4354-4405).
//
// Shape of the contraction: the WEIGHT rows sit on the MMA M side and the tokens
// on the MMA N side (C^T = W * A^T). A CTA tile is 128 weight rows x 256 tokens;
// its fp32 accumulator is 128 TMEM lanes x 256 columns, and the 512 TMEM columns
// hold two of them so the epilogue of one tile overlaps the main loop of the next.
// Both operands are K-major fp16 tiles of 64 columns (one 128-byte swizzle atom)
// brought in by TMA; tcgen05.mma (kind::f16, fp32 accumulate) is issued by a single
// thread and completion is tracked with tcgen05.commit on mbarriers.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM allocator + MMA
// issuer, warps 2..5 = epilogue (tcgen05.ld -> fp32 stores, transposing back to
// C[token][row]; for a fixed token the 32 lanes of a warp write 32 consecutive rows,
// one coalesced 128-byte store).
//
// Operand precision: weights are dequantized exactly to fp32 and rounded once to
// fp16; activations are rounded once to fp16. Each product then carries at most
// 2^-10 relative error and the accumulation is fp32, inside the path's tolerance of
// 1e-3 * sum|w*x| per output.
#include "common.cuh"
#include "gemm.h"

#include <cuda.h>
#include <cuda_fp16.h>

namespace tmc {

namespace {

constexpr int BM = 128;              // weight rows per tile (UMMA M)
constexpr int BN = 256;              // tokens per tile (UMMA N)
constexpr int BK = 64;               // fp16 per tile row: 128 bytes, one swizzle atom
constexpr int kStages = 4;
constexpr int UMMA_K = 16;
constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;
constexpr unsigned long long kWaitNs = 2000000000ull;
constexpr size_t kSmemBytes = (size_t)kStages * STAGE_BYTES + 256 + 1024;   // tiles + barriers + alignment slack

// kind::f16 instruction descriptor: fp32 accumulate, fp16 A and B, both K-major, N=256, M=128
constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_ns() - t0 > kWaitNs) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
// K-major, 128-byte swizzle: rows 128 B apart, 8-row groups 1024 B apart (SBO), LBO unused (1), version 1
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// tmA: weights as fp16 [n_rows][K], box 64 x 128.  tmB: activations as fp16 [m_tok][K], box 64 x 256.
__global__ void __launch_bounds__(kThreads, 1)
gemm_f16_tn(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            float* __restrict__ C, uint32_t ldc, uint32_t m_tok, uint32_t n_rows, uint32_t K, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + (size_t)kStages * STAGE_BYTES);
    uint64_t* empty = full + kStages;
    uint64_t* tfull = empty + kStages;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = (uint32_t*)(tempty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t num_kb = (K + BK - 1) / BK;
    const uint32_t tiles_n = (n_rows + BM - 1) / BM, tiles_m = (m_tok + BN - 1) / BN, tiles = tiles_n * tiles_m;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&tfull[b], 1); mbar_init(&tempty[b], 128); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool dead = false;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (uint32_t tile = blockIdx.x; tile < tiles && !dead; tile += gridDim.x) {
                const int n0 = (int)(tile % tiles_n) * BM, m0 = (int)(tile / tiles_n) * BN;
                for (uint32_t kb = 0; kb < num_kb; ++kb, ++it) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                    if (!mbar_wait(&empty[s], ph ^ 1u)) { dead = true; break; }
                    uint8_t* a = smem + (size_t)s * STAGE_BYTES;
                    mbar_expect_tx(&full[s], STAGE_BYTES);
                    tma_load_2d(a, &tmA, (int)(kb * BK), n0, &full[s]);
                    tma_load_2d(a + A_BYTES, &tmB, (int)(kb * BK), m0, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it = 0, tcount = 0;
            for (uint32_t tile = blockIdx.x; tile < tiles && !dead; tile += gridDim.x, ++tcount) {
                const uint32_t buf = tcount & 1u;
                if (!mbar_wait(&tempty[buf], ((tcount >> 1) & 1u) ^ 1u)) { dead = true; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (uint32_t kb = 0; kb < num_kb; ++kb, ++it) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                    if (!mbar_wait(&full[s], ph)) { dead = true; break; }
                    tc_fence_after();
                    const uint32_t a = smem_u32(smem + (size_t)s * STAGE_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_f16(d_tmem, umma_desc(a + k * UMMA_K * 2), umma_desc(a + A_BYTES + k * UMMA_K * 2), kIdesc,
                                 (kb | (uint32_t)k) ? 1u : 0u);
                    umma_commit(&empty[s]);            // the stage is free once these MMAs have read it
                }
                if (dead) break;
                umma_commit(&tfull[buf]);              // accumulator complete
            }
        }
    } else {
        const uint32_t q = (uint32_t)warp & 3u;        // TMEM lane quarter this warp may read
        uint32_t tcount = 0;
        for (uint32_t tile = blockIdx.x; tile < tiles && !dead; tile += gridDim.x, ++tcount) {
            const uint32_t buf = tcount & 1u;
            const uint32_t n0 = (tile % tiles_n) * BM, m0 = (tile / tiles_n) * BN;
            if (!mbar_wait(&tfull[buf], (tcount >> 1) & 1u)) { dead = true; break; }
            tc_fence_after();
            const uint32_t row = n0 + q * 32 + lane;
            const uint32_t taddr = tmem_base + buf * BN + ((q * 32u) << 16);
            for (uint32_t c0 = 0; c0 < (uint32_t)BN; c0 += 32) {
                if (m0 + c0 >= m_tok) break;            // warp-uniform: whole column block past the last token
                uint32_t v[32];
                tmem_ld32(taddr + c0, v);
                if (row < n_rows) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t m = m0 + c0 + j;
                        if (m < m_tok) C[(size_t)m * ldc + row] = __uint_as_float(v[j]);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&tempty[buf]);
        }
    }
    if (dead) atomicExch(status, 2);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

__global__ void f32_to_f16_rows(const float* __restrict__ src, __half* __restrict__ dst, size_t n4) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const float4 v = reinterpret_cast<const float4*>(src)[i];
    __half2* o = reinterpret_cast<__half2*>(dst) + 2 * i;
    o[0] = __floats2half2_rn(v.x, v.y);
    o[1] = __floats2half2_rn(v.z, v.w);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// fp16 [rows][K] row-major, box 64 x box_rows, 128-byte swizzle, out-of-range reads give zeros
bool make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail("gemm: cuTensorMapEncodeTiled is unavailable");
    const cuuint64_t dims[2] = {K, rows};
    const cuuint64_t strides[1] = {K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("gemm: tensor map encode failed (%d)", (int)r);
    return true;
}

}  // namespace

size_t gemm_workspace_bytes(unsigned M, unsigned N, unsigned K) {
    auto up = [](size_t b) { return (b + 255) / 256 * 256; };
    return up((size_t)N * K * 2) + up((size_t)M * K * 2);
}

bool launch_gemm(const float* A, const uint8_t* W, float* C, unsigned ldc, unsigned M, unsigned N, unsigned K,
                 unsigned dtype, void* workspace, size_t workspace_bytes, cudaStream_t st) {
    const unsigned be = block_elems(dtype);
    if (!be || dtype == DT_F16) return fail("gemm: dtype %u is not a block format", dtype);
    if (!A || !W || !C) return fail("gemm: null pointer");
    if (M == 0 || N == 0) return true;
    if (ldc < N) return fail("gemm: ldc=%u is smaller than N=%u", ldc, N);
    if (K == 0 || K % be) return fail("gemm: K=%u is not a multiple of %u", K, be);
    if (K % 8) return fail("gemm: K must be a multiple of 8");
    if ((uintptr_t)A % 16 || (uintptr_t)C % 4) return fail("gemm: A must be 16-byte aligned");
    if (!workspace || (uintptr_t)workspace % 256 || workspace_bytes < gemm_workspace_bytes(M, N, K))
        return fail("gemm: workspace of %zu bytes (256-byte aligned) required", gemm_workspace_bytes(M, N, K));
    uint8_t* ws = (uint8_t*)workspace;
    __half* Wh = (__half*)ws;
    __half* Ah = (__half*)(ws + ((size_t)N * K * 2 + 255) / 256 * 256);

    if (!launch_dequant_half(W, Wh, N, K, dtype, st)) return false;
    const size_t n4 = (size_t)M * K / 4;
    f32_to_f16_rows<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(A, Ah, n4);
    note_launch();
    if (!check_launch("f32_to_f16_rows")) return false;

    CUtensorMap tmA, tmB;
    if (!make_map(&tmA, Wh, N, K, BM) || !make_map(&tmB, Ah, M, K, BN)) return false;
    static bool attr = false;
    if (!attr) {
        if (cudaFuncSetAttribute(gemm_f16_tn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) != cudaSuccess)
            return check_launch("gemm: shared memory attribute");
        attr = true;
    }
    const unsigned tiles = ((N + BM - 1) / BM) * ((M + BN - 1) / BN);
    unsigned grid = (unsigned)device_sm_count();
    if (grid > tiles) grid = tiles;
    gemm_f16_tn<<<grid, kThreads, kSmemBytes, st>>>(tmA, tmB, C, ldc, M, N, K, device_status_word());
    note_launch();
    return check_launch("gemm_f16_tn");
}

}  // namespace tmc
