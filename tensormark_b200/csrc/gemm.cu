// gemm.cu — prefill GEMM on the 5th-generation tensor cores:  C[M x N] = A[M x K] * W^T.
//
// Replaces the reference's prefill GEMMs (tensormark/metal.h:1387-1449 sgemm_q4,
// 1137-1381 q4_mm_tile*, and the dequantize + MPSMatrixMultiplication path
// 1658-1718) and covers the K-quant LM head for which the reference has no GPU
// GEMM at all (its CPU path dequantizes and calls sgemm, llama.h:4354-4405).
//
// Tile order: the token tiles of one weight-row tile are consecutive tile indices, so the CTAs that run at
// the same time share few weight tiles and every weight tile is fetched from DRAM once (with the weight tile
// index running fastest, a 131 MB fp16 LM head was streamed once per token tile: 974 MB of DRAM reads for a
// 2000 x 32000 x 2048 call, measured).
//
// Shape of the contraction: the WEIGHT rows sit on the MMA M side and the tokens
// on the MMA N side (C^T = W * A^T). A CTA tile is 128 weight rows x 256 tokens;
// its fp32 accumulator is 128 TMEM lanes x 256 columns, and the 512 TMEM columns
// hold two of them so the epilogue of one tile overlaps the main loop of the next.
// Both operands are K-major fp16 tiles of 64 columns (one 128-byte swizzle atom)
// brought in by TMA; tcgen05.mma (kind::f16, fp32 accumulate) is issued by a single
// thread and completion is tracked with tcgen05.commit on mbarriers.
//
// Warp roles of the TMA-fed kernels (256 threads): warps 0, 6, 7 = TMA producers taking the stages in
// turn, warp 1 = TMEM allocator + MMA issuer, warps 2..5 = epilogue (tcgen05.ld -> fp32 stores,
// transposing back to C[token][row]; for a fixed token the 32 lanes of a warp write 32 consecutive
// rows, one coalesced 128-byte store). The in-kernel dequantizing form keeps one TMA producer and adds
// eight converting warps.
//
// Two forms. The default (gemm_f16_tn, and gemm_f16_tn_pair on CTA pairs for calls of many tiles) takes both
// operands by TMA from an fp16 copy that one pre-pass launch writes to the workspace (weights dequantized
// exactly and rounded once, activations rounded once). The other (gemm_q4_tn, TM_GEMM_FUSED=1, Q4_0 only) never materialises the fp16 weights: eight
// producer warps take the rows' 18-byte blocks from a bulk-copied raw ring, turn the nibbles into
// (n - 8) * d with two half2 instructions per pair (the same value the fp32 dequantizer rounded to fp16
// gives) and store them into the stage in the 128-byte-swizzled K-major layout the MMA descriptor
// expects, followed by a proxy fence and an arrive on the stage's barrier; TMA then only carries the
// activations. It is the slower of the two today (its producers wait on their barriers while the tensor
// pipe idles), which is why the pre-pass form is the default.
//
// Operand precision: weights are dequantized exactly to fp32 and rounded once to
// fp16; activations are rounded once to fp16. Each product then carries at most
// 2^-10 relative error and the accumulation is fp32, inside the path's tolerance of
// 1e-3 * sum|w*x| per output.
#include "common.cuh"
#include "gemm.h"

#include <cstdlib>
#include <type_traits>

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
constexpr int kThreads = 192;          // the Q4_0 in-kernel form: producer, MMA issuer, four epilogue warps (+ its dequantizing warps)
constexpr int kProducers = 3;          // TMA-issuing warps of the two TMA-fed kernels (warps 0, 6, 7), taking stages in turn
constexpr int kThreadsTma = 256;
constexpr uint32_t kTmemCols = 512;
constexpr unsigned long long kWaitNs = 2000000000ull;
constexpr int kMaxStages = 8;
constexpr uint32_t kTileRegion = 225u * 1024u;      // operand ring: as many stages of 16 KB + bn x 128 B as fit (4 at bn = 256)
constexpr size_t kSmemBytes = (size_t)kTileRegion + 256 + 1024;              // ring + barriers + alignment slack
static_assert(kStages * STAGE_BYTES <= kTileRegion && kSmemBytes <= 227u * 1024u, "shared memory budget");

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
// One probe, never suspends the thread (try_wait costs ~200 clocks even on a completed phase, test_wait ~80).
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
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
    if (mbar_test(bar, parity)) return true;
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
// The four MMAs of one 64-wide k-block (operand tiles at shared addresses a and b, K advancing 32 bytes per MMA inside
// the swizzle atom) and, issued BEFORE them, a probe of the barrier the next k-block will need; the probe's answer is
// only read after the MMAs are out, so its latency hides behind them. The issuing thread is the kernel's narrowest
// point: a probe, four MMAs and a commit have to fit into the 512 clocks the tensor pipe needs for N = 256.
__device__ __forceinline__ uint64_t umma_desc_at(uint32_t lo, uint32_t k) {       // lo = umma_desc's low word for the tile's start
    constexpr uint32_t hi = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | (uint64_t)(lo + 2u * k);                        // 32 bytes = 2 units of 16
}
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); }
__device__ __forceinline__ bool umma_kblock(uint32_t tmem_d, uint32_t a, uint32_t b, uint32_t idesc, uint32_t acc_first,
                                            uint64_t* next_bar, uint32_t next_parity) {
    const uint32_t la = umma_desc_lo(a), lb = umma_desc_lo(b);
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p, q, t;\n\t"
        "setp.ne.b32 q, %12, 0;\n\t"
        "setp.eq.b32 t, 0, 0;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%13], %14;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], %2, %3, %10, q;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], %4, %5, %10, t;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], %6, %7, %10, t;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], %8, %9, %10, t;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(tmem_d), "l"(umma_desc_at(la, 0)), "l"(umma_desc_at(lb, 0)), "l"(umma_desc_at(la, 1)), "l"(umma_desc_at(lb, 1)),
          "l"(umma_desc_at(la, 2)), "l"(umma_desc_at(lb, 2)), "l"(umma_desc_at(la, 3)), "l"(umma_desc_at(lb, 3)),
          "r"(idesc), "r"(0), "r"(acc_first), "r"(smem_u32(next_bar)), "r"(next_parity)
        : "memory");
    return ok != 0;
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

// tmA: weights as fp16 [n_rows][K], box 64 x 128.  tmB: activations as fp16 [m_tok][K], box 64 x bn.
// bn = tokens per tile (UMMA N): a multiple of 16 up to BN = 256, chosen per call so that the tiles fill whole waves of
// the persistent grid (pick_token_tile). A narrower tile makes a smaller stage, and the ring then holds more of them:
// the bytes in flight per SM, which is what covers the L2 latency, stay the same. The TMEM stride stays 256 columns.
__global__ void __launch_bounds__(kThreadsTma, 1)
gemm_f16_tn(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            float* __restrict__ C, uint32_t ldc, uint32_t m_tok, uint32_t n_rows, uint32_t K, uint32_t bn, uint32_t accumulate,
            int* status, __half* __restrict__ act) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + kTileRegion);
    uint64_t* empty = full + kMaxStages;
    uint64_t* tfull = empty + kMaxStages;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = (uint32_t*)(tempty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t num_kb = (K + BK - 1) / BK;
    const uint32_t tiles_n = (n_rows + BM - 1) / BM, tiles_m = (m_tok + bn - 1) / bn, tiles = tiles_n * tiles_m;
    const uint32_t idesc = (1u << 4) | ((bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);      // kIdesc with N = bn
    const uint32_t stage_bytes = A_BYTES + bn * (uint32_t)(BK * 2);                           // a multiple of 1024
    const uint32_t stages = min((uint32_t)kMaxStages, kTileRegion / stage_bytes);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
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
    // Launched with programmatic stream serialization: everything above (barriers, TMEM) overlaps the pre-pass that
    // writes the fp16 operands; nothing below may start before that kernel has finished.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == 0 || warp >= 6) {
        // Producers. A warp's bulk-tensor copy instruction takes about 300 ns to issue whatever its size and ~25 ns more
        // per active lane (measured: one lane x 4..32 KB boxes, 2..16 stages in flight: 300-320 ns per request; 3 lanes
        // x 16 KB: 358 ns per instruction), so ONE issuing thread per operand fed a stage every ~570 clocks - longer
        // than the stage's four MMAs run. Here a stage's two boxes go out in ONE instruction (lane 0 the weight rows,
        // lane 1 the token rows) and kProducers warps take the stages in turn.
        const uint32_t prod = warp == 0 ? 0u : (uint32_t)warp - 5u;
        const uint32_t my_tiles = tiles > blockIdx.x ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
        const uint32_t total = my_tiles * num_kb;
        for (uint32_t it = prod; it < total; it += kProducers) {
            const uint32_t s = it % stages, ph = (it / stages) & 1u;
            const uint32_t t = it / num_kb, kb = it - t * num_kb, tile = blockIdx.x + t * gridDim.x;
            const int n0 = (int)(tile / tiles_m) * BM, m0 = (int)((tile % tiles_m) * bn);
            if (!__all_sync(0xffffffffu, mbar_wait(&empty[s], ph ^ 1u))) { dead = true; break; }
            uint8_t* a = smem + (size_t)s * stage_bytes;
            if (lane == 0) mbar_expect_tx(&full[s], stage_bytes);
            __syncwarp();
            if (lane < 2)
                tma_load_2d(lane == 0 ? a : a + A_BYTES, lane == 0 ? &tmA : &tmB, (int)(kb * BK), lane == 0 ? n0 : m0, &full[s]);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t s = 0, ph = 0, tcount = 0;
            bool ready = false;                                  // what the probe issued with the previous k-block said
            for (uint32_t tile = blockIdx.x; tile < tiles && !dead; tile += gridDim.x, ++tcount) {
                const uint32_t buf = tcount & 1u;
                if (!mbar_wait(&tempty[buf], ((tcount >> 1) & 1u) ^ 1u)) { dead = true; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (!ready && !mbar_wait(&full[s], ph)) { dead = true; break; }
                    tc_fence_after();
                    const uint32_t a = smem_u32(smem) + s * stage_bytes;
                    uint32_t s1 = s + 1, ph1 = ph;
                    if (s1 == stages) { s1 = 0; ph1 ^= 1u; }
                    ready = umma_kblock(d_tmem, a, a + A_BYTES, idesc, kb ? 1u : 0u, &full[s1], ph1);
                    umma_commit(&empty[s]);            // the stage is free once these MMAs have read it
                    s = s1; ph = ph1;
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
            const uint32_t n0 = (tile / tiles_m) * BM, m0 = (tile % tiles_m) * bn;
            if (!mbar_wait(&tfull[buf], (tcount >> 1) & 1u)) { dead = true; break; }
            tc_fence_after();
            const uint32_t row = n0 + q * 32 + lane;
            const uint32_t taddr = tmem_base + buf * BN + ((q * 32u) << 16);
            for (uint32_t c0 = 0; c0 < bn; c0 += 32) {
                if (m0 + c0 >= m_tok) break;            // warp-uniform: whole column block past the last token
                uint32_t v[32];
                tmem_ld32(taddr + c0, v);               // a 16-column remainder reads 16 stale columns of the buffer: masked below
                if (act) {
                    // Gated FFN: weight row 2f is gate row f and row 2f + 1 is up row f, so the two lanes of a pair hold
                    // gate and up of the same f for the same 32 tokens. They trade halves - the even lane keeps tokens
                    // 0-15 and gets their up values, the odd lane keeps 16-31 and gets their gate values - and each
                    // writes silu(gate) * up for its 16 tokens as fp16 into act[token][f] (ldc = F): the gate|up values
                    // never reach memory. Same expression and rounding as the separate kernel this replaces.
                    const bool odd = lane & 1;
                    float res[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float mine_lo = __uint_as_float(v[j]), mine_hi = __uint_as_float(v[16 + j]);
                        const float got = __shfl_xor_sync(0xffffffffu, odd ? mine_lo : mine_hi, 1);
                        const float g = odd ? got : mine_lo, u = odd ? mine_hi : got;
                        res[j] = g / (1.0f + expf(-g)) * u;
                    }
                    if (row < n_rows) {
                        const uint32_t f = row >> 1, cb = c0 + (odd ? 16u : 0u);
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const uint32_t m = m0 + cb + j;
                            if (cb + j < bn && m < m_tok) act[(size_t)m * ldc + f] = __float2half_rn(res[j]);
                        }
                    }
                    continue;
                }
                if (row < n_rows) {
                    if (accumulate) {                   // C += A W^T (a residual add folded in): all 32 old values are requested before the first is used
                        float old[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const uint32_t m = m0 + c0 + j;
                            old[j] = (c0 + j < bn && m < m_tok) ? __ldcg(C + (size_t)m * ldc + row) : 0.f;
                        }
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(old[j] + __uint_as_float(v[j]));
                    }
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t m = m0 + c0 + j;
                        if (c0 + j < bn && m < m_tok) C[(size_t)m * ldc + row] = __uint_as_float(v[j]);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&tempty[buf]);
        }
    }
    if (dead) *(volatile int*)status = 2;
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}


// ---- the same GEMM on CTA pairs (tcgen05 cta_group::2) ----------------------------------------------------------
// Two CTAs of a cluster share one 256 x bn tile: each loads its own 128 weight rows and HALF of the token rows; the
// MMA, issued by the even CTA for both, reads the token rows out of both CTAs' shared memory, and each CTA's 128 x bn
// accumulator lands in its own TMEM. Two things are gained. Operand delivery: 16 KB + bn x 64 B per CTA and 64 columns
// of K instead of 16 KB + bn x 128 B (at bn = 256 the one-CTA kernel asks L2 for 94 bytes per clock and SM, about what
// one SM gets; its MMA thread then waits for operands a fifth of the time). Issue rate: one issued MMA drives both
// SMs' tensor pipes, and a stage here is two swizzle atoms of K (128 columns), so the issuing thread spends one
// barrier probe and one commit per EIGHT MMAs.
// Same-GPU A/B against the one-CTA kernel, 2000 tokens: 6 % faster on the 32000 x 2048 head (14 waves of tiles),
// 1-2 % slower on 5632 x 2048 and 2048 x 5632 (three waves, one wave); the launcher takes this kernel from four waves
// of pair tiles.
//
// Barriers: the loads of both CTAs count on the EVEN CTA's full[s] (a TMA load may signal the pair's other CTA);
// empty[s] and tfull[buf] are raised in both CTAs by one multicast commit; the epilogue warps of both CTAs arrive
// on the even CTA's tempty[buf] (256 arrivals). Every wait is bounded like the single-CTA kernel's.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {      // shared::cta address -> shared::cluster address in CTA `rank`
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
// The MMAs of TWO consecutive stages (eight MMAs) behind probes of the two stages after them: per 64 columns of K the
// issuing thread spends half a probe and four MMA issues. Bit 0 of the result: bar0's phase is complete, bit 1: bar1's.
__device__ __forceinline__ uint32_t umma_kblock2_pair(uint32_t tmem_d, uint32_t a0, uint32_t b0, uint32_t a1, uint32_t b1, uint32_t idesc,
                                                      uint32_t acc_first, uint64_t* bar0, uint32_t parity0, uint64_t* bar1, uint32_t parity1) {
    const uint32_t la = umma_desc_lo(a0), lb = umma_desc_lo(b0), la1 = umma_desc_lo(a1), lb1 = umma_desc_lo(b1);
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p0, p1, q, t;\n\t.reg .u32 r0, r1;\n\t"
        "setp.ne.b32 q, %20, 0;\n\t"
        "setp.eq.b32 t, 0, 0;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p0, [%21], %22;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p1, [%23], %24;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], %2, %3, %18, {%19, %19, %19, %19, %19, %19, %19, %19}, q;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], %4, %5, %18, {%19, %19, %19, %19, %19, %19, %19, %19}, t;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], %6, %7, %18, {%19, %19, %19, %19, %19, %19, %19, %19}, t;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], %8, %9, %18, {%19, %19, %19, %19, %19, %19, %19, %19}, t;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], %10, %11, %18, {%19, %19, %19, %19, %19, %19, %19, %19}, t;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], %12, %13, %18, {%19, %19, %19, %19, %19, %19, %19, %19}, t;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], %14, %15, %18, {%19, %19, %19, %19, %19, %19, %19, %19}, t;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], %16, %17, %18, {%19, %19, %19, %19, %19, %19, %19, %19}, t;\n\t"
        "selp.u32 r0, 1, 0, p0;\n\t"
        "selp.u32 r1, 2, 0, p1;\n\t"
        "or.b32 %0, r0, r1;\n\t}"
        : "=r"(ok)
        : "r"(tmem_d), "l"(umma_desc_at(la, 0)), "l"(umma_desc_at(lb, 0)), "l"(umma_desc_at(la, 1)), "l"(umma_desc_at(lb, 1)),
          "l"(umma_desc_at(la, 2)), "l"(umma_desc_at(lb, 2)), "l"(umma_desc_at(la, 3)), "l"(umma_desc_at(lb, 3)),
          "l"(umma_desc_at(la1, 0)), "l"(umma_desc_at(lb1, 0)), "l"(umma_desc_at(la1, 1)), "l"(umma_desc_at(lb1, 1)),
          "l"(umma_desc_at(la1, 2)), "l"(umma_desc_at(lb1, 2)), "l"(umma_desc_at(la1, 3)), "l"(umma_desc_at(lb1, 3)),
          "r"(idesc), "r"(0), "r"(acc_first), "r"(smem_u32(bar0)), "r"(parity0), "r"(smem_u32(bar1)), "r"(parity1)
        : "memory");
    return ok;
}
// One stage (a tile's odd last k-block), one probe.
__device__ __forceinline__ uint32_t umma_kblock_pair(uint32_t tmem_d, uint32_t a, uint32_t b, uint32_t idesc, uint32_t acc_first,
                                                     uint64_t* next_bar, uint32_t next_parity) {
    const uint32_t la = umma_desc_lo(a), lb = umma_desc_lo(b);
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p, q, t;\n\t"
        "setp.ne.b32 q, %12, 0;\n\t"
        "setp.eq.b32 t, 0, 0;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%13], %14;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], %2, %3, %10, {%11, %11, %11, %11, %11, %11, %11, %11}, q;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], %4, %5, %10, {%11, %11, %11, %11, %11, %11, %11, %11}, t;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], %6, %7, %10, {%11, %11, %11, %11, %11, %11, %11, %11}, t;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], %8, %9, %10, {%11, %11, %11, %11, %11, %11, %11, %11}, t;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(tmem_d), "l"(umma_desc_at(la, 0)), "l"(umma_desc_at(lb, 0)), "l"(umma_desc_at(la, 1)), "l"(umma_desc_at(lb, 1)),
          "l"(umma_desc_at(la, 2)), "l"(umma_desc_at(lb, 2)), "l"(umma_desc_at(la, 3)), "l"(umma_desc_at(lb, 3)),
          "r"(idesc), "r"(0), "r"(acc_first), "r"(smem_u32(next_bar)), "r"(next_parity)
        : "memory");
    return ok;
}
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {        // arrives on `bar` at this offset in both CTAs
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(both) : "memory");
}

// tmA: box 64 x 128 of the fp16 weights. tmB: box 64 x bn/2 of the fp16 activations. bn: tokens per pair tile, a
// multiple of 32 up to 256. Grid: an even number of CTAs, clusters of two. A stage per CTA: two weight atoms (2 x 16 KB),
// then two token atoms (2 x bn/2 x 128 B); three stages at bn = 256.
__global__ void __launch_bounds__(kThreadsTma, 1)
gemm_f16_tn_pair(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 float* __restrict__ C, uint32_t ldc, uint32_t m_tok, uint32_t n_rows, uint32_t K, uint32_t bn, uint32_t accumulate,
                 int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);     // the same offset in both CTAs
    uint64_t* full = (uint64_t*)(smem + kTileRegion);
    uint64_t* empty = full + kMaxStages;
    uint64_t* tfull = empty + kMaxStages;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = (uint32_t*)(tempty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                     // 0: issues the MMAs and owns full[] and tempty[]
    const uint32_t pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const uint32_t half = bn >> 1;
    const uint32_t num_kb = (K + BK - 1) / BK;
    const uint32_t tiles_n = (n_rows + 2 * BM - 1) / (2 * BM), tiles_m = (m_tok + bn - 1) / bn, tiles = tiles_n * tiles_m;
    const uint32_t idesc = (1u << 4) | ((bn >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);   // M = 256 over the pair, N = bn
    const uint32_t stage_bytes = A_BYTES + half * (uint32_t)(BK * 2);                            // per CTA; a multiple of 1024
    const uint32_t stages = min((uint32_t)kMaxStages, kTileRegion / stage_bytes);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&tfull[b], 1); mbar_init(&tempty[b], 256); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();                                          // both CTAs' barriers exist before either signals the other
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool dead = false;
    asm volatile("griddepcontrol.wait;" ::: "memory");           // the pre-pass has written the fp16 operands

    if (warp == 0 || warp >= 6) {
        // Producers, as in gemm_f16_tn: a stage's two boxes go out in one instruction, kProducers warps take the stages in turn.
        const uint32_t prod = warp == 0 ? 0u : (uint32_t)warp - 5u;
        const uint32_t my_tiles = tiles > pair ? (tiles - pair + npairs - 1) / npairs : 0u;
        const uint32_t total = my_tiles * num_kb;
        for (uint32_t it = prod; it < total; it += kProducers) {
            const uint32_t s = it % stages, ph = (it / stages) & 1u;
            const uint32_t t = it / num_kb, kb = it - t * num_kb, tile = pair + t * npairs;
            const int n0 = (int)((tile / tiles_m) * 2 * BM + rank * BM), m0 = (int)((tile % tiles_m) * bn + rank * half);
            if (!__all_sync(0xffffffffu, mbar_wait(&empty[s], ph ^ 1u))) { dead = true; break; }
            uint8_t* a = smem + (size_t)s * stage_bytes;
            const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
            if (lane == 0 && rank == 0) mbar_expect_tx(&full[s], 2 * stage_bytes);
            __syncwarp();
            if (lane < 2)                                                // rows or tokens past the end arrive as zeros
                tma_load_2d_pair(lane == 0 ? a : a + A_BYTES, lane == 0 ? &tmA : &tmB, (int)(kb * BK), lane == 0 ? n0 : m0, bar);
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            uint32_t s = 0, ph = 0, tcount = 0, ready = 0;      // ready: bit 0 / 1 = stage s / the one after it was complete when last probed
            auto next = [&](uint32_t& st, uint32_t& p) { if (++st == stages) { st = 0; p ^= 1u; } };
            for (uint32_t tile = pair; tile < tiles && !dead; tile += npairs, ++tcount) {
                const uint32_t buf = tcount & 1u;
                if (!mbar_wait(&tempty[buf], ((tcount >> 1) & 1u) ^ 1u)) { dead = true; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (uint32_t kb = 0; kb < num_kb; kb += 2) {
                    const bool two = kb + 1 < num_kb;
                    uint32_t s1 = s, ph1 = ph;
                    next(s1, ph1);
                    if (!(ready & 1u) && !mbar_wait(&full[s], ph)) { dead = true; break; }
                    if (two && !(ready & 2u) && !mbar_wait(&full[s1], ph1)) { dead = true; break; }
                    tc_fence_after();
                    const uint32_t a0 = smem_u32(smem) + s * stage_bytes, a1 = smem_u32(smem) + s1 * stage_bytes;
                    if (two) {
                        uint32_t s2 = s1, ph2 = ph1;
                        next(s2, ph2);
                        uint32_t s3 = s2, ph3 = ph2;
                        next(s3, ph3);
                        ready = umma_kblock2_pair(d_tmem, a0, a0 + A_BYTES, a1, a1 + A_BYTES, idesc, kb ? 1u : 0u, &full[s2], ph2, &full[s3], ph3);
                        umma_commit_pair(&empty[s]);
                        umma_commit_pair(&empty[s1]);
                        s = s2; ph = ph2;
                    } else {
                        ready = umma_kblock_pair(d_tmem, a0, a0 + A_BYTES, idesc, kb ? 1u : 0u, &full[s1], ph1);
                        umma_commit_pair(&empty[s]);
                        s = s1; ph = ph1;
                    }
                }
                if (dead) break;
                umma_commit_pair(&tfull[buf]);
            }
        }
    } else {
        const uint32_t q = (uint32_t)warp & 3u;
        uint32_t tcount = 0;
        for (uint32_t tile = pair; tile < tiles && !dead; tile += npairs, ++tcount) {
            const uint32_t buf = tcount & 1u;
            const uint32_t n0 = (tile / tiles_m) * 2 * BM + rank * BM, m0 = (tile % tiles_m) * bn;
            if (!mbar_wait(&tfull[buf], (tcount >> 1) & 1u)) { dead = true; break; }
            tc_fence_after();
            const uint32_t row = n0 + q * 32 + lane;
            const uint32_t taddr = tmem_base + buf * BN + ((q * 32u) << 16);
            for (uint32_t c0 = 0; c0 < bn; c0 += 32) {
                if (m0 + c0 >= m_tok) break;
                uint32_t v[32];
                tmem_ld32(taddr + c0, v);
                if (row < n_rows) {
                    if (accumulate) {
                        float old[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const uint32_t m = m0 + c0 + j;
                            old[j] = m < m_tok ? __ldcg(C + (size_t)m * ldc + row) : 0.f;
                        }
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(old[j] + __uint_as_float(v[j]));
                    }
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t m = m0 + c0 + j;
                        if (m < m_tok) C[(size_t)m * ldc + row] = __uint_as_float(v[j]);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive_cluster(map_to_cta(smem_u32(&tempty[buf]), 0));
        }
    }
    if (dead) *(volatile int*)status = 2;
    tc_fence_before();
    cluster_sync_all();                  // neither CTA leaves, or frees its TMEM, while the other may still signal or read it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}


// ---- Q4_0: dequantizing producer --------------------------------------------------------------
constexpr int kDqWarps = 8;                      // two sets of four warps, alternating k-blocks; a thread owns one tile row
constexpr int kThreadsQ4 = kThreads + kDqWarps * 32;

// Four consecutive nibble codes (the low nibbles of the four bytes of `q4`, already masked) as two
// half2 of (n - 8) * d.
__device__ __forceinline__ void q4_quad(uint32_t q4, __half2 d2, uint32_t& o01, uint32_t& o23) {
    const __half2 k1032 = __half2half2(__ushort_as_half((unsigned short)0x6408));      // 1032.0
    uint32_t a = __byte_perm(q4, 0x64646464u, 0x5140), b = __byte_perm(q4, 0x64646464u, 0x7362);   // 1024 + n in each half
    __half2 ha = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&a), k1032), d2);
    __half2 hb = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&b), k1032), d2);
    o01 = *reinterpret_cast<uint32_t*>(&ha); o23 = *reinterpret_cast<uint32_t*>(&hb);
}
// One Q4_0 block (d, 16 code bytes in Q[0..3]) -> 32 fp16 = chunks c0 .. c0+3 of the row, swizzled.
// Byte j of a block holds weight 2j in its low nibble and weight 2j+1 in its high nibble
// (tensormark/quant.h:194-200), so one 32-bit word is eight consecutive weights = one 16-byte chunk.
__device__ __forceinline__ void q4_block_to_stage(uint8_t* row_base, uint32_t r7, uint32_t c0, uint32_t dbits, const uint32_t (&Q)[4]) {
    const __half2 d2 = __half2half2(__ushort_as_half((unsigned short)dbits));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t lo = Q[i] & 0x0F0F0F0Fu, hi = (Q[i] >> 4) & 0x0F0F0F0Fu;
        const uint32_t p01 = __byte_perm(lo, hi, 0x5140), p23 = __byte_perm(lo, hi, 0x7362);   // codes in weight order
        uint4 o;
        q4_quad(p01, d2, o.x, o.y);
        q4_quad(p23, d2, o.z, o.w);
        *reinterpret_cast<uint4*>(row_base + (((c0 + i) ^ r7) << 4)) = o;
    }
}

// Raw blocks reach the producers through shared memory: a row's bytes for four k-blocks (8 blocks, 144 bytes)
// arrive by one bulk copy per row, 128 rows per raw stage. Reading them from global memory with one 4-byte
// load per lane instead costs a cache-tag lookup per lane and load, which took longer than the MMAs.
//
// Three rings, each with its own barriers, so that the depth of each follows what it has to hide:
//   activations (TMA, 32 KB per k-block)  kStagesB = 4   L2 latency at the MMA's consumption rate
//   fp16 weights (written by producers)   kStagesA = 3   only the conversion itself
//   raw blocks (bulk copies, 18 KB per 4 k-blocks) kRaw = 2, refilled as soon as the rows are in registers
constexpr int kStagesB = 4, kStagesA = 3, kRaw = 2;
constexpr uint32_t RAW_ROW = 144, RAW_BYTES = BM * RAW_ROW;
constexpr size_t kSmemBytesQ4 = (size_t)kStagesB * B_BYTES + (size_t)kStagesA * A_BYTES + (size_t)kRaw * RAW_BYTES + 256 + 1024;
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// W: Q4_0 blocks [n_rows][K/32], rows 16-byte aligned; tmB: activations as fp16 [m_tok][K], box 64 x 256. K % 256 == 0.
__global__ void __launch_bounds__(kThreadsQ4, 1)
gemm_q4_tn(const uint8_t* __restrict__ W, uint32_t row_bytes, const __grid_constant__ CUtensorMap tmB,
           float* __restrict__ C, uint32_t ldc, uint32_t m_tok, uint32_t n_rows, uint32_t K, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* bbuf = smem;                                          // kStagesB x 32 KB, 1024-byte aligned
    uint8_t* abuf = bbuf + (size_t)kStagesB * B_BYTES;             // kStagesA x 16 KB, 1024-byte aligned
    uint8_t* raw = abuf + (size_t)kStagesA * A_BYTES;
    uint64_t* bfull = (uint64_t*)(raw + (size_t)kRaw * RAW_BYTES);
    uint64_t* bempty = bfull + kStagesB;
    uint64_t* afull = bempty + kStagesB;
    uint64_t* aempty = afull + kStagesA;
    uint64_t* tfull = aempty + kStagesA;
    uint64_t* tempty = tfull + 2;
    uint64_t* rfull = tempty + 2;
    uint64_t* rempty = rfull + kRaw;
    uint32_t* tmem_slot = (uint32_t*)(rempty + kRaw);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t num_kb = K / BK;
    const uint32_t tiles_n = (n_rows + BM - 1) / BM, tiles_m = (m_tok + BN - 1) / BN, tiles = tiles_n * tiles_m;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStagesB; ++s) { mbar_init(&bfull[s], 1); mbar_init(&bempty[s], 1); }
        // a weight stage is full when the four warps that convert this k-block have arrived
        for (int s = 0; s < kStagesA; ++s) { mbar_init(&afull[s], 4); mbar_init(&aempty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&tfull[b], 1); mbar_init(&tempty[b], 128); }
        // a raw stage is full when its 128 row copies have landed (each loader thread arrives with its bytes) and
        // free again when all eight producer warps have taken their rows into registers
        for (int s = 0; s < kRaw; ++s) { mbar_init(&rfull[s], BM); mbar_init(&rempty[s], kDqWarps); }
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
                const int m0 = (int)(tile % tiles_m) * BN;
                for (uint32_t kb = 0; kb < num_kb; ++kb, ++it) {
                    const uint32_t s = it % kStagesB, ph = (it / kStagesB) & 1u;
                    if (!mbar_wait(&bempty[s], ph ^ 1u)) { dead = true; break; }
                    mbar_expect_tx(&bfull[s], B_BYTES);
                    tma_load_2d(bbuf + (size_t)s * B_BYTES, &tmB, (int)(kb * BK), m0, &bfull[s]);
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
                    const uint32_t sb = it % kStagesB, phb = (it / kStagesB) & 1u;
                    const uint32_t sa = it % kStagesA, pha = (it / kStagesA) & 1u;
                    if (!mbar_wait(&afull[sa], pha) || !mbar_wait(&bfull[sb], phb)) { dead = true; break; }
                    tc_fence_after();
                    const uint32_t a = smem_u32(abuf + (size_t)sa * A_BYTES), b = smem_u32(bbuf + (size_t)sb * B_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_f16(d_tmem, umma_desc(a + k * UMMA_K * 2), umma_desc(b + k * UMMA_K * 2), kIdesc,
                                 (kb | (uint32_t)k) ? 1u : 0u);
                    umma_commit(&aempty[sa]);          // both stages are free once these MMAs have read them
                    umma_commit(&bempty[sb]);
                }
                if (dead) break;
                umma_commit(&tfull[buf]);
            }
        }
    } else if (warp < 6) {
        const uint32_t q = (uint32_t)warp & 3u;        // TMEM lane quarter this warp may read
        uint32_t tcount = 0;
        for (uint32_t tile = blockIdx.x; tile < tiles && !dead; tile += gridDim.x, ++tcount) {
            const uint32_t buf = tcount & 1u;
            const uint32_t n0 = (tile / tiles_m) * BM, m0 = (tile % tiles_m) * BN;
            if (!mbar_wait(&tfull[buf], (tcount >> 1) & 1u)) { dead = true; break; }
            tc_fence_after();
            const uint32_t row = n0 + q * 32 + lane;
            const uint32_t taddr = tmem_base + buf * BN + ((q * 32u) << 16);
            for (uint32_t c0 = 0; c0 < (uint32_t)BN; c0 += 32) {
                if (m0 + c0 >= m_tok) break;
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
    } else {
        // ---- dequantizing producers: two sets of four warps, thread r of a set owns tile row r.
        // The CTA's k-blocks, in pipeline order, form groups of four (K % 256 == 0, so a group never straddles
        // tiles). Group G sits in raw stage G % kRaw. Of a group's four k-blocks set 0 converts the first and third,
        // set 1 the others. Set 0's threads also request the rows: groups 0 and 1 up front, then group G + 2 as
        // soon as group G has been converted (its raw stage is free once all eight warps hold it in registers).
        const uint32_t set = (uint32_t)(warp - 6) >> 2, r = ((uint32_t)(warp - 6) & 3u) * 32u + (uint32_t)lane;
        const uint32_t r7 = r & 7u;
        const uint32_t groups_per_tile = num_kb / 4;
        uint32_t my_tiles = 0;
        for (uint32_t t = blockIdx.x; t < tiles; t += gridDim.x) ++my_tiles;
        const uint32_t ngroups = my_tiles * groups_per_tile;
        auto issue = [&](uint32_t G) -> bool {
            if (G >= ngroups) return true;
            const uint32_t rs = G % kRaw, rph = (G / kRaw) & 1u;
            if (!mbar_wait(&rempty[rs], rph ^ 1u)) { dead = true; return false; }
            const uint32_t tile = blockIdx.x + (G / groups_per_tile) * gridDim.x, g = G % groups_per_tile;
            const uint32_t row = (tile / tiles_m) * BM + r;
            if (row < n_rows) {
                mbar_expect_tx(&rfull[rs], RAW_ROW);
                bulk_g2s(raw + (size_t)rs * RAW_BYTES + r * RAW_ROW, W + (size_t)row * row_bytes + (size_t)g * RAW_ROW, RAW_ROW, &rfull[rs]);
            } else {
                mbar_arrive(&rfull[rs]);                           // past the last row: nothing to copy, zeros are produced below
            }
            return true;
        };
        if (set == 0) { if (issue(0)) (void)issue(1); }
        for (uint32_t G = 0; G < ngroups && !dead; ++G) {
            const uint32_t rs = G % kRaw, rph = (G / kRaw) & 1u;
            if (!mbar_wait(&rfull[rs], rph)) { dead = true; break; }
            const uint32_t tile = blockIdx.x + (G / groups_per_tile) * gridDim.x;
            const bool live = (tile / tiles_m) * BM + r < n_rows;
            uint32_t w[36];                                        // this row's 144 bytes: 9 conflict-free 16-byte reads
            const uint4* src = reinterpret_cast<const uint4*>(raw + (size_t)rs * RAW_BYTES + r * RAW_ROW);
#pragma unroll
            for (int i = 0; i < 9; ++i) {
                const uint4 v = live ? src[i] : make_uint4(0u, 0u, 0u, 0u);
                w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&rempty[rs]);
            // k-blocks (2j + set) of the group, with compile-time register offsets (set is warp-uniform)
            auto item = [&](auto KQ) -> bool {
                constexpr uint32_t kq = decltype(KQ)::value;
                const uint32_t it = G * 4u + kq;
                const uint32_t s = it % kStagesA, ph = (it / kStagesA) & 1u;
                if (!mbar_wait(&aempty[s], ph ^ 1u)) { dead = true; return false; }
                uint8_t* row_base = abuf + (size_t)s * A_BYTES + (r >> 3) * 1024u + r7 * 128u;
                uint32_t Q[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) Q[i] = __byte_perm(w[9 * kq + i], w[9 * kq + i + 1], 0x5432);     // block 0: code bytes 2 .. 17
                q4_block_to_stage(row_base, r7, 0, w[9 * kq] & 0xFFFFu, Q);
#pragma unroll
                for (int i = 0; i < 4; ++i) Q[i] = w[9 * kq + 5 + i];                                           // block 1: d at byte 18, codes 20 .. 35
                q4_block_to_stage(row_base, r7, 4, w[9 * kq + 4] >> 16, Q);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic-proxy stores -> visible to the MMA's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(&afull[s]);
                return true;
            };
            using I0 = std::integral_constant<uint32_t, 0>; using I1 = std::integral_constant<uint32_t, 1>;
            using I2 = std::integral_constant<uint32_t, 2>; using I3 = std::integral_constant<uint32_t, 3>;
            if (set == 0) { if (!item(I0{}) || !item(I2{})) break; if (!issue(G + 2)) break; }
            else { if (!item(I1{}) || !item(I3{})) break; }
        }
    }
    if (dead) *(volatile int*)status = 2;
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

// Items per thread of the pre-pass kernels: a block covers 256 x kPrepItems consecutive items, each thread taking
// every 256th, all loads requested before the first is used (with one item per thread the launches were 9632 and
// 36000 short blocks that spent more time being scheduled than working).
constexpr int kPrepItems = 4;

__device__ __forceinline__ void round_activations(const float* __restrict__ A, __half* __restrict__ Ah, size_t n4, size_t first) {
    float4 v[kPrepItems];
#pragma unroll
    for (int j = 0; j < kPrepItems; ++j) {
        const size_t i = first + (size_t)j * 256;
        if (i < n4) v[j] = __ldg(reinterpret_cast<const float4*>(A) + i);
    }
#pragma unroll
    for (int j = 0; j < kPrepItems; ++j) {
        const size_t i = first + (size_t)j * 256;
        if (i < n4) {
            const __half2 lo = __floats2half2_rn(v[j].x, v[j].y), hi = __floats2half2_rn(v[j].z, v[j].w);
            reinterpret_cast<uint2*>(Ah)[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
        }
    }
}

// Both operand conversions of the Q4_0 pre-pass form in one launch. Blocks [0, blocks_w) turn weights into fp16:
// one item per 32-bit word of codes = eight consecutive weights = one 16-byte store, consecutive threads consecutive
// words, with the same two-instruction-per-pair arithmetic as the producer warps of gemm_q4_tn (the exact (n - 8) * d
// rounded once to fp16). The remaining blocks round the activations.
__global__ void __launch_bounds__(256) prepass_q4_f16(const uint8_t* __restrict__ W, uint32_t row_bytes, __half* __restrict__ Wh,
                                                      uint32_t N, uint32_t K, const float* __restrict__ A, __half* __restrict__ Ah,
                                                      size_t n4, uint32_t blocks_w) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");        // the GEMM may set itself up meanwhile
    if (blockIdx.x < blocks_w) {
        const uint32_t wpr = K / 8;                                         // words per row
        const uint64_t total = (uint64_t)N * wpr, first = (uint64_t)blockIdx.x * (256 * kPrepItems) + threadIdx.x;
        uint32_t dbits[kPrepItems], q[kPrepItems];
#pragma unroll
        for (int j = 0; j < kPrepItems; ++j) {
            const uint64_t idx = first + (uint64_t)j * 256;
            if (idx < total) {
                const uint32_t row = (uint32_t)(idx / wpr), w = (uint32_t)(idx % wpr), blk = w >> 2, i = w & 3u;
                const unsigned short* p = reinterpret_cast<const unsigned short*>(W + (size_t)row * row_bytes + (size_t)blk * 18u);
                dbits[j] = __ldg(p);
                q[j] = (uint32_t)__ldg(p + 1 + 2 * i) | ((uint32_t)__ldg(p + 2 + 2 * i) << 16);
            }
        }
#pragma unroll
        for (int j = 0; j < kPrepItems; ++j) {
            const uint64_t idx = first + (uint64_t)j * 256;
            if (idx < total) {
                const __half2 d2 = __half2half2(__ushort_as_half((unsigned short)dbits[j]));
                const uint32_t lo = q[j] & 0x0F0F0F0Fu, hi = (q[j] >> 4) & 0x0F0F0F0Fu;
                const uint32_t p01 = __byte_perm(lo, hi, 0x5140), p23 = __byte_perm(lo, hi, 0x7362);
                uint4 o;
                q4_quad(p01, d2, o.x, o.y);
                q4_quad(p23, d2, o.z, o.w);
                reinterpret_cast<uint4*>(Wh)[idx] = o;                      // rows are K / 8 sixteen-byte words long: word idx of the whole matrix
            }
        }
    } else {
        round_activations(A, Ah, n4, (size_t)(blockIdx.x - blocks_w) * (256 * kPrepItems) + threadIdx.x);
    }
}

// The same for Q6_K: one item per eight consecutive weights (they share the super-block scale, the sub-block scale,
// the nibble half and the high-bit pair position), d * sc and then * (q - 32) in fp32 (both products are exact, as in
// tmq::dequantize_row_q6_k, tensormark/quant.h:338-365), rounded once to fp16, one 16-byte store.
__global__ void __launch_bounds__(256) prepass_q6k_f16(const uint8_t* __restrict__ W, uint32_t row_bytes, __half* __restrict__ Wh,
                                                       uint32_t N, uint32_t K, const float* __restrict__ A, __half* __restrict__ Ah,
                                                       size_t n4, uint32_t blocks_w) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (blockIdx.x < blocks_w) {
        const uint32_t gpr = K / 8;                                         // groups of eight per row
        const uint64_t total = (uint64_t)N * gpr, first = (uint64_t)blockIdx.x * (256 * kPrepItems) + threadIdx.x;
        uint32_t qlw[kPrepItems][2], qhw[kPrepItems][2], jj[kPrepItems];
        float ds[kPrepItems];
#pragma unroll
        for (int it = 0; it < kPrepItems; ++it) {
            const uint64_t idx = first + (uint64_t)it * 256;
            if (idx < total) {
                const uint32_t row = (uint32_t)(idx / gpr), t = (uint32_t)(idx % gpr), k = t * 8;
                const uint32_t e = k & 255u, h = e >> 7, j = (e >> 5) & 3u, l0 = e & 31u;
                const uint8_t* b = W + (size_t)row * row_bytes + (size_t)(k >> 8) * 210u;
                const unsigned short* ql = reinterpret_cast<const unsigned short*>(b + 64 * h + 32 * (j & 1u) + l0);
                const unsigned short* qh = reinterpret_cast<const unsigned short*>(b + 128 + 32 * h + l0);
                const uint32_t dbits = __ldg(reinterpret_cast<const unsigned short*>(b + 208));
                const int sc = (int)(int8_t)__ldg(b + 192 + 8 * h + 2 * j + (l0 >> 4));
                ds[it] = __fmul_rn(__half2float(__ushort_as_half((unsigned short)dbits)), __int2float_rn(sc));
                jj[it] = j;
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    qlw[it][w] = (uint32_t)__ldg(ql + 2 * w) | ((uint32_t)__ldg(ql + 2 * w + 1) << 16);
                    qhw[it][w] = (uint32_t)__ldg(qh + 2 * w) | ((uint32_t)__ldg(qh + 2 * w + 1) << 16);
                }
            }
        }
#pragma unroll
        for (int it = 0; it < kPrepItems; ++it) {
            const uint64_t idx = first + (uint64_t)it * 256;
            if (idx < total) {
                const uint32_t j = jj[it];
                uint32_t o[4];
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    const uint32_t nib = ((j & 2u) ? (qlw[it][w] >> 4) : qlw[it][w]) & 0x0F0F0F0Fu;
                    const uint32_t code = nib | (((qhw[it][w] >> (2 * j)) & 0x03030303u) << 4);          // four codes 0..63
                    const float w0 = __fmul_rn(ds[it], __int2float_rn((int)(code & 255u) - 32));
                    const float w1 = __fmul_rn(ds[it], __int2float_rn((int)((code >> 8) & 255u) - 32));
                    const float w2 = __fmul_rn(ds[it], __int2float_rn((int)((code >> 16) & 255u) - 32));
                    const float w3 = __fmul_rn(ds[it], __int2float_rn((int)(code >> 24) - 32));
                    const __half2 a = __floats2half2_rn(w0, w1), c = __floats2half2_rn(w2, w3);
                    o[2 * w] = *reinterpret_cast<const uint32_t*>(&a);
                    o[2 * w + 1] = *reinterpret_cast<const uint32_t*>(&c);
                }
                reinterpret_cast<uint4*>(Wh)[idx] = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    } else {
        round_activations(A, Ah, n4, (size_t)(blockIdx.x - blocks_w) * (256 * kPrepItems) + threadIdx.x);
    }
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

// Tokens per tile. The persistent grid runs the tiles in waves of one per SM, and a call's time is (waves) x (time of
// a tile), so a tile width that fills the last wave beats the widest one: 2000 tokens against 5632 rows are 352 tiles
// of 256 tokens = 2.38 waves run as 3, but 440 tiles of 208 tokens = 2.97 waves. A tile's time is modelled as
// 128 + bn (the kernel is bound by operand delivery: 128 weight rows + bn token rows per k-block). Widths below 64
// are only taken when the whole batch is narrower.
unsigned pick_token_tile(unsigned M, unsigned N, unsigned sms) {
    static const int forced = [] { const char* e = std::getenv("TM_GEMM_BN"); return e && *e ? std::atoi(e) : 0; }();   // A/B knob
    if (forced >= 16 && forced <= BN && forced % 16 == 0) return (unsigned)forced;
    const unsigned rt = (N + BM - 1) / BM;
    if (M <= 64) return (M + 15) / 16 * 16;
    unsigned best = BN;
    unsigned long long best_cost = ~0ull;
    for (unsigned bn = BN; bn >= 64; bn -= 16) {
        const unsigned long long tiles = (unsigned long long)rt * ((M + bn - 1) / bn), waves = (tiles + sms - 1) / sms;
        const unsigned long long cost = waves * (128 + bn);
        if (cost < best_cost) { best_cost = cost; best = bn; }
    }
    return best;
}

// The same for the CTA-pair kernel: 256 weight rows x bn tokens per pair of SMs, bn a multiple of 32. Per k-block a
// CTA takes 16 KB + bn x 64 B from L2 at 64 B per clock (256 + bn clocks) while the pair's MMAs run about 2.1 clocks
// per token column; the slower of the two is the tile's time.
unsigned pick_token_tile_pair(unsigned M, unsigned N, unsigned sms) {
    static const int forced = [] { const char* e = std::getenv("TM_GEMM_BN"); return e && *e ? std::atoi(e) : 0; }();
    if (forced >= 32 && forced <= BN && forced % 32 == 0) return (unsigned)forced;
    const unsigned rt = (N + 2 * BM - 1) / (2 * BM), pairs = sms / 2 ? sms / 2 : 1;
    if (M <= 64) return (M + 31) / 32 * 32;
    unsigned best = BN;
    unsigned long long best_cost = ~0ull;
    for (unsigned bn = BN; bn >= 64; bn -= 32) {
        const unsigned long long tiles = (unsigned long long)rt * ((M + bn - 1) / bn), waves = (tiles + pairs - 1) / pairs;
        const unsigned long long l2 = 256 + bn, mma = (unsigned long long)bn * 21 / 10;
        const unsigned long long cost = waves * (l2 > mma ? l2 : mma);
        if (cost < best_cost) { best_cost = cost; best = bn; }
    }
    return best;
}

}  // namespace

// The TMA-fed kernels over fp16 operands that are in place (or being written by the launch just before this one):
// weights Wh [N][K], activations Ah [M][K].
// act (instead of C): the weights are gate and up rows interleaved and the output is act[M][ldc] = silu(gate) * up in
// fp16 (the one-SM kernel's fused epilogue; such calls do not take the CTA-pair kernel).
static bool launch_tiles(const __half* Wh, const __half* Ah, float* C, unsigned ldc, unsigned M, unsigned N, unsigned K, cudaStream_t st,
                         bool accumulate = false, __half* act = nullptr) {
    CUtensorMap tmA, tmB;
    // Two SMs per tile (gemm_f16_tn_pair) where it measured faster: four or more waves of pair tiles. TM_GEMM_PAIR=0
    // keeps one SM per tile everywhere, TM_GEMM_PAIR=1 pairs wherever there are 256 weight rows.
    static const int pair_mode = [] { const char* e = std::getenv("TM_GEMM_PAIR"); return e && *e ? std::atoi(e) : -1; }();
    const unsigned sms = (unsigned)device_sm_count();
    const unsigned bn2 = pick_token_tile_pair(M, N, sms);
    const unsigned long long pair_tiles = (unsigned long long)((N + 2 * BM - 1) / (2 * BM)) * ((M + bn2 - 1) / bn2);
    const bool paired = !act && N >= 2 * BM && sms >= 2 && (pair_mode == 1 || (pair_mode < 0 && pair_tiles >= 4ull * (sms / 2)));
    if (paired) {
        if (!make_map(&tmB, Ah, M, K, bn2 / 2) || !make_map(&tmA, Wh, N, K, BM)) return false;
        static bool attr2 = false;
        if (!attr2) {
            if (cudaFuncSetAttribute(gemm_f16_tn_pair, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) != cudaSuccess)
                return check_launch("gemm: shared memory attribute");
            attr2 = true;
        }
        const unsigned tiles2 = ((N + 2 * BM - 1) / (2 * BM)) * ((M + bn2 - 1) / bn2);
        const unsigned pairs = sms / 2 < tiles2 ? sms / 2 : tiles2;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(kThreadsTma); cfg.dynamicSmemBytes = kSmemBytes; cfg.stream = st;
        cudaLaunchAttribute at[2];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        at[1].id = cudaLaunchAttributeClusterDimension;
        at[1].val.clusterDim.x = 2; at[1].val.clusterDim.y = 1; at[1].val.clusterDim.z = 1;
        cfg.attrs = at; cfg.numAttrs = 2;
        if (cudaLaunchKernelEx(&cfg, gemm_f16_tn_pair, tmA, tmB, C, (uint32_t)ldc, (uint32_t)M, (uint32_t)N, (uint32_t)K, (uint32_t)bn2,
                               accumulate ? 1u : 0u, device_status_word()) != cudaSuccess)
            return check_launch("gemm_f16_tn_pair");
        note_launch();
        return check_launch("gemm_f16_tn_pair");
    }
    const unsigned bn = pick_token_tile(M, N, sms);
    if (!make_map(&tmB, Ah, M, K, bn) || !make_map(&tmA, Wh, N, K, BM)) return false;
    static bool attr = false;
    if (!attr) {
        if (cudaFuncSetAttribute(gemm_f16_tn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) != cudaSuccess)
            return check_launch("gemm: shared memory attribute");
        attr = true;
    }
    const unsigned tiles = ((N + BM - 1) / BM) * ((M + bn - 1) / bn);
    unsigned grid = sms;
    if (grid > tiles) grid = tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kThreadsTma); cfg.dynamicSmemBytes = kSmemBytes; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, gemm_f16_tn, tmA, tmB, C, (uint32_t)ldc, (uint32_t)M, (uint32_t)N, (uint32_t)K, (uint32_t)bn,
                           accumulate ? 1u : 0u, device_status_word(), act) != cudaSuccess)
        return check_launch("gemm_f16_tn");
    note_launch();
    return check_launch("gemm_f16_tn");
}

// fp16 copy of a block-quantized tensor: the weight half of launch_gemm's pre-pass, for callers that keep it (the prefill
// layer stack converts its static weights once instead of once per call).
bool launch_weights_f16(const uint8_t* W, void* Wh_out, unsigned N, unsigned K, unsigned dtype, cudaStream_t st) {
    const unsigned be = block_elems(dtype);
    if (!be || dtype == DT_F16) return fail("gemm: dtype %u is not a block format", dtype);
    if (!W || !Wh_out || (uintptr_t)Wh_out % 16) return fail("gemm: bad pointer for the fp16 weights");
    if (N == 0) return true;
    if (K == 0 || K % be || K % 8) return fail("gemm: K=%u is not a multiple of %u and of 8", K, be);
    __half* Wh = (__half*)Wh_out;
    const uint32_t row_bytes = (K / be) * block_bytes(dtype);
    const unsigned per = 256 * kPrepItems;
    const unsigned blocks_w = (unsigned)(((uint64_t)N * (K / 8) + per - 1) / per);
    if (dtype == DT_Q4_0 && (uintptr_t)W % 2 == 0 && row_bytes % 2 == 0) {
        prepass_q4_f16<<<blocks_w, 256, 0, st>>>(W, row_bytes, Wh, N, K, nullptr, nullptr, 0, blocks_w);
    } else if (dtype == DT_Q6_K && (uintptr_t)W % 2 == 0 && row_bytes % 2 == 0) {
        prepass_q6k_f16<<<blocks_w, 256, 0, st>>>(W, row_bytes, Wh, N, K, nullptr, nullptr, 0, blocks_w);
    } else {
        return launch_dequant_half(W, Wh, N, K, dtype, st);
    }
    note_launch();
    return check_launch("weights_f16");
}

// Both operands already fp16 (weights from launch_weights_f16, activations written as fp16 by the kernel that made
// them): no pre-pass and no workspace at all. accumulate: C += A W^T.
bool launch_gemm_hh(const void* Ah, const void* Wh, float* C, unsigned ldc, unsigned M, unsigned N, unsigned K, bool accumulate, cudaStream_t st) {
    if (!Ah || !Wh || !C) return fail("gemm: null pointer");
    if (M == 0 || N == 0) return true;
    if (ldc < N) return fail("gemm: ldc=%u is smaller than N=%u", ldc, N);
    if (K == 0 || K % 8) return fail("gemm: K must be a multiple of 8");
    if ((uintptr_t)Ah % 16 || (uintptr_t)C % 4 || (uintptr_t)Wh % 16) return fail("gemm: the fp16 operands must be 16-byte aligned");
    return launch_tiles((const __half*)Wh, (const __half*)Ah, C, ldc, M, N, K, st, accumulate);
}

// act[M][F] = silu(A Wg^T) * (A Wu^T) in fp16, where Wgu [2 F][K] holds gate row f at row 2f and up row f at row 2f + 1.
bool launch_gemm_hh_silu_mul(const void* Ah, const void* Wgu, void* act, unsigned M, unsigned F, unsigned K, cudaStream_t st) {
    if (!Ah || !Wgu || !act) return fail("gemm: null pointer");
    if (M == 0 || F == 0) return true;
    if (K == 0 || K % 8) return fail("gemm: K must be a multiple of 8");
    if ((uintptr_t)Ah % 16 || (uintptr_t)act % 2 || (uintptr_t)Wgu % 16) return fail("gemm: the fp16 operands must be 16-byte aligned");
    return launch_tiles((const __half*)Wgu, (const __half*)Ah, nullptr, F, M, 2 * F, K, st, false, (__half*)act);
}

size_t gemm_f16w_workspace_bytes(unsigned M, unsigned K) { return ((size_t)M * K * 2 + 255) / 256 * 256; }

// The GEMM against weights that are already fp16 (launch_weights_f16): only the activations are rounded per call.
bool launch_gemm_f16w(const float* A, const void* Wh, float* C, unsigned ldc, unsigned M, unsigned N, unsigned K,
                      void* workspace, size_t workspace_bytes, cudaStream_t st) {
    if (!A || !Wh || !C) return fail("gemm: null pointer");
    if (M == 0 || N == 0) return true;
    if (ldc < N) return fail("gemm: ldc=%u is smaller than N=%u", ldc, N);
    if (K == 0 || K % 8) return fail("gemm: K must be a multiple of 8");
    if ((uintptr_t)A % 16 || (uintptr_t)C % 4 || (uintptr_t)Wh % 16) return fail("gemm: A and the fp16 weights must be 16-byte aligned");
    if (!workspace || (uintptr_t)workspace % 256 || workspace_bytes < gemm_f16w_workspace_bytes(M, K))
        return fail("gemm: workspace of %zu bytes (256-byte aligned) required", gemm_f16w_workspace_bytes(M, K));
    __half* Ah = (__half*)workspace;
    const size_t n4 = (size_t)M * K / 4;
    f32_to_f16_rows<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(A, Ah, n4);
    note_launch();
    if (!check_launch("f32_to_f16_rows")) return false;
    return launch_tiles((const __half*)Wh, Ah, C, ldc, M, N, K, st);
}

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

    // Q4_0 with K a multiple of 256 and 16-byte aligned rows can be dequantized inside the GEMM (gemm_q4_tn).
    // TM_GEMM_FUSED=1 selects it; the default is the pre-pass, which is the faster of the two today
    // (2000 x 5632 x 2048: 72 us for pre-passes + TMA-fed kernel against 77 us for the producer-fed kernel,
    // whose tensor pipe is 30 % busy with the producers stalled on their barriers).
    static const bool allow_fused = [] { const char* e = std::getenv("TM_GEMM_FUSED"); return e && *e == '1'; }();
    const uint32_t row_bytes = (K / be) * block_bytes(dtype);
    const bool fused = allow_fused && dtype == DT_Q4_0 && K % 256 == 0 && (uintptr_t)W % 16 == 0 && row_bytes % 16 == 0;
    const size_t n4 = (size_t)M * K / 4;
    if (!fused && dtype == DT_Q4_0 && K % 8 == 0 && (uintptr_t)W % 2 == 0 && row_bytes % 2 == 0) {
        const unsigned per = 256 * kPrepItems;
        const unsigned blocks_w = (unsigned)(((uint64_t)N * (K / 8) + per - 1) / per), blocks_a = (unsigned)((n4 + per - 1) / per);
        prepass_q4_f16<<<blocks_w + blocks_a, 256, 0, st>>>(W, row_bytes, Wh, N, K, A, Ah, n4, blocks_w);
        note_launch();
        if (!check_launch("prepass_q4_f16")) return false;
    } else if (dtype == DT_Q6_K && (uintptr_t)W % 2 == 0 && row_bytes % 2 == 0) {
        const unsigned per = 256 * kPrepItems;
        const unsigned blocks_w = (unsigned)(((uint64_t)N * (K / 8) + per - 1) / per), blocks_a = (unsigned)((n4 + per - 1) / per);
        prepass_q6k_f16<<<blocks_w + blocks_a, 256, 0, st>>>(W, row_bytes, Wh, N, K, A, Ah, n4, blocks_w);
        note_launch();
        if (!check_launch("prepass_q6k_f16")) return false;
    } else {
        if (!fused && !launch_dequant_half(W, Wh, N, K, dtype, st)) return false;
        f32_to_f16_rows<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(A, Ah, n4);
        note_launch();
        if (!check_launch("f32_to_f16_rows")) return false;
    }

    if (fused) {
        CUtensorMap tmB;
        if (!make_map(&tmB, Ah, M, K, BN)) return false;
        static bool attr4 = false;
        if (!attr4) {
            if (cudaFuncSetAttribute(gemm_q4_tn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytesQ4) != cudaSuccess)
                return check_launch("gemm: shared memory attribute");
            attr4 = true;
        }
        const unsigned tiles4 = ((N + BM - 1) / BM) * ((M + BN - 1) / BN);
        unsigned grid4 = (unsigned)device_sm_count();
        if (grid4 > tiles4) grid4 = tiles4;
        gemm_q4_tn<<<grid4, kThreadsQ4, kSmemBytesQ4, st>>>(W, row_bytes, tmB, C, ldc, M, N, K, device_status_word());
        note_launch();
        return check_launch("gemm_q4_tn");
    }
    return launch_tiles(Wh, Ah, C, ldc, M, N, K, st);
}

}  // namespace tmc
