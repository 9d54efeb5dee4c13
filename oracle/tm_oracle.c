/* oracle/tm_oracle.c — CPU restatement of the reference's quantized-weight matmul path.
 *
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE. Only the test-suite, the smoke check
 * and the benchmark's CPU-baseline legs load this library; the CUDA library
 * never links or calls it.
 *
 * Every function restates, in plain C, what the reference computes on a
 * non-Apple, non-NEON host, and names the reference lines it follows. It is
 * pinned two ways: (1) libtm_ref.so (built next to it from the reference's own
 * tensormark/quant.h, see ref_wrap.cpp) must agree bit for bit with tmo_dequant
 * and the fp16 conversions on random blocks; (2) the committed golden vectors
 * under tests/golden were produced by that reference build.
 *
 * Build with -ffp-contract=off: the reference writes q*d + m, d1*q - m1 and
 * d*sc*q as separate fp32 operations and the bit-exact dequant gate depends on
 * them staying separate.
 */
#include <math.h>
#include <pthread.h>
#include <stdatomic.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define TMO_API __attribute__((visibility("default")))

/* ---- fp16 <-> fp32 (tensormark/quant.h:58-70, 120-146) ------------------- */
static float bits_f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t f_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

TMO_API float tmo_fp16_to_fp32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t ex = (h >> 10) & 0x1fu, man = h & 0x3ffu;
    if (ex == 0) {
        if (man == 0) return bits_f(sign);
        return bits_f(sign | (f_bits((float)man * 0x1p-24f) & 0x7fffffffu));
    }
    if (ex == 31) return bits_f(sign | 0x7f800000u | (man << 13));
    return bits_f(sign | ((ex + 112u) << 23) | (man << 13));
}

TMO_API uint16_t tmo_fp32_to_fp16(float f) {
    uint32_t x = f_bits(f), sign = (x >> 16) & 0x8000u;
    uint32_t e32 = (x >> 23) & 0xffu, man = x & 0x7fffffu;
    if (e32 == 0xffu) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0u));
    int e = (int)e32 - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7c00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        uint32_t m = man | 0x800000u;
        int sh = 14 - e;
        uint32_t q = m >> sh, rem = m & ((1u << sh) - 1u), tie = 1u << (sh - 1);
        if (rem > tie || (rem == tie && (q & 1u))) q++;
        return (uint16_t)(sign | q);
    }
    uint32_t r = man >> 13, rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) r++;
    if (r >> 10) { e++; r = 0; }
    return (uint16_t)(sign | ((uint32_t)e << 10) | (r & 0x3ffu));
}

static uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* ---- geometry (tensormark/tmq.h:83-115) ---------------------------------- */
TMO_API int tmo_block_elems(int dtype) {
    switch (dtype) { case 0: case 1: case 4: case 9: return 32; case 5: case 6: case 8: return 256; case 7: return 128; default: return 0; }
}
TMO_API int tmo_block_bytes(int dtype) {
    switch (dtype) { case 0: case 7: return 34; case 1: case 9: return 18; case 4: return 20; case 5: return 176; case 6: return 210; case 8: return 144; default: return 0; }
}

/* ---- dequantizers --------------------------------------------------------- */
/* Q8_0, quant.h:194-200: w = (float)q * d */
static void deq_q8_0(const uint8_t* b, float* x) {
    float d = tmo_fp16_to_fp32(rd16(b));
    for (int i = 0; i < 32; i++) x[i] = (float)(int8_t)b[2 + i] * d;
}
/* Q4_0, quant.h:397-408: interleaved nibbles, w = (float)(n - 8) * d */
static void deq_q4_0(const uint8_t* b, float* x) {
    float d = tmo_fp16_to_fp32(rd16(b));
    for (int j = 0; j < 16; j++) {
        int n0 = b[2 + j] & 0x0f, n1 = b[2 + j] >> 4;
        x[2 * j] = (float)(n0 - 8) * d;
        x[2 * j + 1] = (float)(n1 - 8) * d;
    }
}
/* Q4_1, quant.h:267-277: split nibbles, w = (float)n * d + m (two roundings) */
static void deq_q4_1(const uint8_t* b, float* x) {
    float d = tmo_fp16_to_fp32(rd16(b)), m = tmo_fp16_to_fp32(rd16(b + 2));
    for (int j = 0; j < 16; j++) {
        float a = (float)(b[4 + j] & 0x0fu) * d;
        float c = (float)(b[4 + j] >> 4) * d;
        x[j] = a + m;
        x[j + 16] = c + m;
    }
}
/* 6-bit pair unpack, quant.h:256-264 */
static void scale_min(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
    if (j < 4) { *d = q[j] & 63u; *m = q[j + 4] & 63u; }
    else {
        *d = (uint8_t)((q[j + 4] & 0x0fu) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}
/* Q4_K, quant.h:282-301: four groups of 64; low nibbles = sub-block 2g, high nibbles = 2g+1; w = d1*code - m1 */
static void deq_q4_k(const uint8_t* b, float* x) {
    float d = tmo_fp16_to_fp32(rd16(b)), dm = tmo_fp16_to_fp32(rd16(b + 2));
    const uint8_t *scales = b + 4, *qs = b + 16;
    for (int g = 0; g < 4; g++) {
        uint8_t sc, mn;
        scale_min(2 * g, scales, &sc, &mn);
        float d1 = d * (float)sc, m1 = dm * (float)mn;
        scale_min(2 * g + 1, scales, &sc, &mn);
        float d2 = d * (float)sc, m2 = dm * (float)mn;
        for (int j = 0; j < 32; j++) {
            uint8_t packed = qs[32 * g + j];
            float p1 = d1 * (float)(packed & 0x0fu), p2 = d2 * (float)(packed >> 4);
            x[64 * g + j] = p1 - m1;
            x[64 * g + 32 + j] = p2 - m2;
        }
    }
}
/* Q5_K, quant.h:304-330: d1 = d*sc, m1 = dmin*mn, w = d1*code - m1 */
static void deq_q5_k(const uint8_t* b, float* x) {
    float d = tmo_fp16_to_fp32(rd16(b)), dm = tmo_fp16_to_fp32(rd16(b + 2));
    const uint8_t *scales = b + 4, *qh = b + 16, *ql = b + 48;
    uint8_t u1 = 1, u2 = 2;
    int is = 0;
    for (int j = 0; j < 256; j += 64) {
        uint8_t sc, mn;
        scale_min(is, scales, &sc, &mn);
        float d1 = d * (float)sc, m1 = dm * (float)mn;
        scale_min(is + 1, scales, &sc, &mn);
        float d2 = d * (float)sc, m2 = dm * (float)mn;
        for (int l = 0; l < 32; l++) {
            float p = d1 * (float)((ql[l] & 0x0fu) + ((qh[l] & u1) ? 16 : 0));
            x[j + l] = p - m1;
        }
        for (int l = 0; l < 32; l++) {
            float p = d2 * (float)((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0));
            x[j + 32 + l] = p - m2;
        }
        ql += 32; is += 2; u1 = (uint8_t)(u1 << 2); u2 = (uint8_t)(u2 << 2);
    }
}
/* Q6_K, quant.h:338-365: w = (d * sc) * code, evaluated left to right */
static void deq_q6_k(const uint8_t* b, float* x) {
    const uint8_t *ql = b, *qh = b + 128;
    const int8_t* sc = (const int8_t*)(b + 192);
    float d = tmo_fp16_to_fp32(rd16(b + 208));
    for (int half = 0; half < 256; half += 128) {
        for (int l = 0; l < 32; l++) {
            int is = l / 16;
            int q1 = (int)((ql[l] & 0x0fu) | (((qh[l] >> 0) & 3u) << 4)) - 32;
            int q2 = (int)((ql[l + 32] & 0x0fu) | (((qh[l] >> 2) & 3u) << 4)) - 32;
            int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3u) << 4)) - 32;
            int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3u) << 4)) - 32;
            float s0 = d * (float)sc[is + 0], s2 = d * (float)sc[is + 2];
            float s4 = d * (float)sc[is + 4], s6 = d * (float)sc[is + 6];
            x[l] = s0 * (float)q1;
            x[l + 32] = s2 * (float)q2;
            x[l + 64] = s4 * (float)q3;
            x[l + 96] = s6 * (float)q4;
        }
        x += 128; ql += 64; qh += 32; sc += 8;
    }
}

/* n weights (whole blocks) of `dtype`; returns 0 on a bad argument. */
/* TQ2 (container dtype 7), quant.h:507-515 dequantize_ternary: 128 two-bit codes, four per byte, low bits first;
 * x[j] = (float)(code - 1) * d. */
static void deq_tq2(const uint8_t* b, float* x) {
    float d = tmo_fp16_to_fp32(rd16(b));
    for (int j = 0; j < 128; j++) x[j] = (float)((int)((b[2 + (j >> 2)] >> (2 * (j & 3))) & 3) - 1) * d;
}
/* GGUF's own Q4_0 (container dtype 9), llama.h:4588-4597: the Q4_0 block with split nibbles,
 * x[j] = d * ((qs[j] & 15) - 8), x[j + 16] = d * ((qs[j] >> 4) - 8). */
static void deq_gguf_q4_0(const uint8_t* b, float* x) {
    float d = tmo_fp16_to_fp32(rd16(b));
    for (int j = 0; j < 16; j++) {
        x[j] = d * (float)((b[2 + j] & 15) - 8);
        x[j + 16] = d * (float)((b[2 + j] >> 4) - 8);
    }
}
/* The converter's nibble reorder (convert_gguf.cpp:124-135): a split-nibble block as the container's interleaved
 * Q4_0 block with the same scale and the same 32 codes; dequantizing either gives the same bits. */
TMO_API void tmo_q4_split_to_interleaved(const uint8_t* src, uint8_t* dst, size_t nblocks) {
    for (size_t b = 0; b < nblocks; b++, src += 18, dst += 18) {
        uint8_t code[32];
        for (int j = 0; j < 16; j++) { code[j] = src[2 + j] & 15; code[j + 16] = src[2 + j] >> 4; }
        dst[0] = src[0]; dst[1] = src[1];
        for (int j = 0; j < 16; j++) dst[2 + j] = (uint8_t)(code[2 * j] | (code[2 * j + 1] << 4));
    }
}

TMO_API int tmo_dequant(int dtype, const void* blocks, float* out, size_t n) {
    int be = tmo_block_elems(dtype), bb = tmo_block_bytes(dtype);
    if (!be || n % (size_t)be) return 0;
    const uint8_t* p = (const uint8_t*)blocks;
    for (size_t b = 0; b < n / (size_t)be; b++, p += bb, out += be) {
        switch (dtype) {
            case 0: deq_q8_0(p, out); break;
            case 1: deq_q4_0(p, out); break;
            case 4: deq_q4_1(p, out); break;
            case 5: deq_q5_k(p, out); break;
            case 7: deq_tq2(p, out); break;
            case 8: deq_q4_k(p, out); break;
            case 9: deq_gguf_q4_0(p, out); break;
            default: deq_q6_k(p, out); break;
        }
    }
    return 1;
}

/* ---- GEMV ------------------------------------------------------------------
 * Q8_0 / Q4_0: tensormark/llama.h:1873-1897 (Llama::qgemv): per 32-block fp32
 * partial sum of code*x in element order, times the block scale, added to an
 * fp32 row accumulator. Q4_1 / Q5_K / Q6_K: what the reference does on a host
 * without NEON (llama.h:3774-3783 with dequant_row_kq 4567-4628): dequantize the
 * row to fp32, then a dense fp32 dot (cblas_sgemv there, a plain loop here).
 * Rows [o0, o1) only; y is the base pointer (gemv_pool.h:253-264). */
static void gemv_rows(int dtype, const uint8_t* W, const float* x, float* y, int n_in, int o0, int o1) {
    int be = tmo_block_elems(dtype), bb = tmo_block_bytes(dtype);
    size_t row_bytes = (size_t)(n_in / be) * (size_t)bb;
    if (dtype == 0 || dtype == 1) {
        size_t nb = (size_t)n_in / 32;
        for (int o = o0; o < o1; o++) {
            const uint8_t* r = W + (size_t)o * row_bytes;
            float acc = 0.f;
            for (size_t b = 0; b < nb; b++) {
                const uint8_t* blk = r + b * (size_t)bb;
                float d = tmo_fp16_to_fp32(rd16(blk)), s = 0.f;
                const float* xb = x + b * 32;
                if (dtype == 0) {
                    for (int i = 0; i < 32; i++) s += (float)(int8_t)blk[2 + i] * xb[i];
                } else {
                    for (int j = 0; j < 16; j++)
                        s += (float)((blk[2 + j] & 0xF) - 8) * xb[2 * j] + (float)((blk[2 + j] >> 4) - 8) * xb[2 * j + 1];
                }
                acc += s * d;
            }
            y[o] = acc;
        }
        return;
    }
    float* w = (float*)malloc(sizeof(float) * (size_t)n_in);
    for (int o = o0; o < o1; o++) {
        tmo_dequant(dtype, W + (size_t)o * row_bytes, w, (size_t)n_in);
        float acc = 0.f;
        for (int k = 0; k < n_in; k++) acc += w[k] * x[k];
        y[o] = acc;
    }
    free(w);
}

TMO_API int tmo_gemv(int dtype, const void* W, const float* x, float* y, int n_out, int n_in) {
    int be = tmo_block_elems(dtype);
    if (!be || n_in % be) return 0;
    gemv_rows(dtype, (const uint8_t*)W, x, y, n_in, 0, n_out);
    return 1;
}

/* fp64 companion used as the tolerance reference: y64[o] = sum_k w_k x_k and
 * yabs[o] = sum_k |w_k x_k| with w the dequantized fp32 weights. */
TMO_API int tmo_gemv_f64(int dtype, const void* W, const float* x, double* y64, double* yabs, int n_out, int n_in) {
    int be = tmo_block_elems(dtype), bb = tmo_block_bytes(dtype);
    if (!be || n_in % be) return 0;
    size_t row_bytes = (size_t)(n_in / be) * (size_t)bb;
    float* w = (float*)malloc(sizeof(float) * (size_t)n_in);
    for (int o = 0; o < n_out; o++) {
        tmo_dequant(dtype, (const uint8_t*)W + (size_t)o * row_bytes, w, (size_t)n_in);
        double a = 0, s = 0;
        for (int k = 0; k < n_in; k++) { double p = (double)w[k] * (double)x[k]; a += p; s += fabs(p); }
        y64[o] = a; if (yabs) yabs[o] = s;
    }
    free(w);
    return 1;
}

/* ---- row-chunk pool (tensormark/gemv_pool.h:253-264, 296-315) -------------
 * The reference splits a GEMV into 64-row chunks claimed from an atomic counter
 * by the pool's threads, the caller included; its workers are persistent: a job is
 * published under a generation counter, the workers wake, claim chunks until none
 * is left, and the caller (which claims chunks too) waits for the last one. Restated
 * with pthreads: workers are created on first use and sleep on a condition variable
 * between jobs. One job at a time (the reference's dispatch is single-caller too). */
typedef struct {
    int dtype; const uint8_t* W; const float* x; float* y; int n_in, n_out, chunk;
    atomic_ulong next;
} gemv_job;

static void gemv_claim(gemv_job* j) {
    for (;;) {
        unsigned long start = atomic_fetch_add(&j->next, 1ul) * (unsigned long)j->chunk;
        if (start >= (unsigned long)j->n_out) break;
        unsigned long end = start + (unsigned long)j->chunk;
        if (end > (unsigned long)j->n_out) end = (unsigned long)j->n_out;
        gemv_rows(j->dtype, j->W, j->x, j->y, j->n_in, (int)start, (int)end);
    }
}

#define TMO_POOL_MAX 256
static struct {
    pthread_mutex_t mu; pthread_cond_t wake, idle;
    pthread_t th[TMO_POOL_MAX];
    int nthreads;                 /* workers alive */
    unsigned long generation;     /* bumped per job */
    int want;                     /* workers asked to join the current job */
    int joined, finished;         /* of the current job */
    gemv_job* job;
} g_pool = { PTHREAD_MUTEX_INITIALIZER, PTHREAD_COND_INITIALIZER, PTHREAD_COND_INITIALIZER, {0}, 0, 0ul, 0, 0, 0, NULL };

static void* pool_worker(void* arg) {
    (void)arg;
    unsigned long seen = 0;
    pthread_mutex_lock(&g_pool.mu);
    for (;;) {
        while (g_pool.generation == seen || g_pool.joined >= g_pool.want) {
            if (g_pool.generation != seen) seen = g_pool.generation;   /* job full: sit this one out */
            pthread_cond_wait(&g_pool.wake, &g_pool.mu);
        }
        seen = g_pool.generation;
        g_pool.joined++;
        gemv_job* j = g_pool.job;
        pthread_mutex_unlock(&g_pool.mu);
        gemv_claim(j);
        pthread_mutex_lock(&g_pool.mu);
        if (++g_pool.finished == g_pool.want) pthread_cond_signal(&g_pool.idle);
    }
    return NULL;
}

TMO_API int tmo_gemv_mt(int dtype, const void* W, const float* x, float* y, int n_out, int n_in, int threads) {
    int be = tmo_block_elems(dtype);
    if (!be || n_in % be || threads < 1) return 0;
    gemv_job j = { dtype, (const uint8_t*)W, x, y, n_in, n_out, 64 };
    atomic_init(&j.next, 0ul);
    int helpers = threads - 1;
    if (helpers > TMO_POOL_MAX) helpers = TMO_POOL_MAX;
    pthread_mutex_lock(&g_pool.mu);
    while (g_pool.nthreads < helpers) {
        if (pthread_create(&g_pool.th[g_pool.nthreads], NULL, pool_worker, NULL) != 0) break;
        pthread_detach(g_pool.th[g_pool.nthreads]);
        g_pool.nthreads++;
    }
    if (helpers > g_pool.nthreads) helpers = g_pool.nthreads;
    g_pool.job = &j; g_pool.want = helpers; g_pool.joined = 0; g_pool.finished = 0;
    g_pool.generation++;
    if (helpers) pthread_cond_broadcast(&g_pool.wake);
    pthread_mutex_unlock(&g_pool.mu);
    gemv_claim(&j);                                     /* the caller works too */
    pthread_mutex_lock(&g_pool.mu);
    while (g_pool.finished < g_pool.want) pthread_cond_wait(&g_pool.idle, &g_pool.mu);
    g_pool.job = NULL; g_pool.want = 0;
    pthread_mutex_unlock(&g_pool.mu);
    return 1;
}

/* ---- GEMM: C[M x N] = A[M x K] * W^T ---------------------------------------
 * tensormark/llama.h:4354-4445 (gemm_w): dequantize the whole tensor to an fp32
 * scratch, then cblas_sgemm(RowMajor, NoTrans, Trans). The BLAS is replaced by a
 * plain fp32 dot per output in k order. Token rows [m0, m1). */
typedef struct { const float* A; const float* Wf; float* C; int M, N, K; atomic_int next; } gemm_job;

static void* gemm_worker(void* p) {
    gemm_job* j = (gemm_job*)p;
    for (;;) {
        int m = atomic_fetch_add(&j->next, 1);
        if (m >= j->M) break;
        const float* a = j->A + (size_t)m * j->K;
        for (int n = 0; n < j->N; n++) {
            const float* w = j->Wf + (size_t)n * j->K;
            float acc = 0.f;
            for (int k = 0; k < j->K; k++) acc += a[k] * w[k];
            j->C[(size_t)m * j->N + n] = acc;
        }
    }
    return NULL;
}

TMO_API int tmo_gemm(int dtype, const void* W, const float* A, float* C, int M, int N, int K, int threads) {
    int be = tmo_block_elems(dtype);
    if (!be || K % be || threads < 1) return 0;
    float* Wf = (float*)malloc(sizeof(float) * (size_t)N * (size_t)K);
    if (!Wf) return 0;
    tmo_dequant(dtype, W, Wf, (size_t)N * (size_t)K);
    gemm_job j = { A, Wf, C, M, N, K };
    atomic_init(&j.next, 0);
    pthread_t* t = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)threads);
    int started = 0;
    for (int i = 1; i < threads; i++) if (pthread_create(&t[started], NULL, gemm_worker, &j) == 0) started++;
    gemm_worker(&j);
    for (int i = 0; i < started; i++) pthread_join(t[i], NULL);
    free(t); free(Wf);
    return 1;
}

/* fp64 reference and sum of |a w| for sampled outputs: idx holds ns pairs (m, n). */
TMO_API int tmo_gemm_f64_samples(int dtype, const void* W, const float* A, int N, int K,
                                 const int* idx, int ns, double* y64, double* yabs) {
    int be = tmo_block_elems(dtype), bb = tmo_block_bytes(dtype);
    if (!be || K % be) return 0;
    (void)N;
    size_t row_bytes = (size_t)(K / be) * (size_t)bb;
    float* w = (float*)malloc(sizeof(float) * (size_t)K);
    for (int s = 0; s < ns; s++) {
        int m = idx[2 * s], n = idx[2 * s + 1];
        tmo_dequant(dtype, (const uint8_t*)W + (size_t)n * row_bytes, w, (size_t)K);
        const float* a = A + (size_t)m * K;
        double acc = 0, ab = 0;
        for (int k = 0; k < K; k++) { double p = (double)a[k] * (double)w[k]; acc += p; ab += fabs(p); }
        y64[s] = acc; yabs[s] = ab;
    }
    free(w);
    return 1;
}

/* ---- decode-chain glue -------------------------------------------------------
 * RMSNorm, tensormark/llama.h:5614-5618 (scalar branch). */
TMO_API void tmo_rmsnorm(const float* x, const float* wt, float* out, int n, float eps) {
    float ss = 0.f;
    for (int i = 0; i < n; i++) ss += x[i] * x[i];
    float r = 1.f / sqrtf(ss / n + eps);
    for (int i = 0; i < n; i++) out[i] = x[i] * r * wt[i];
}

/* RoPE on one head, llama.h:5640-5657: inverse frequency pow(theta, -2j/dh) in
 * fp32 (gdn.h:242-252), phase = (float)pos * inv, pairs (j, j + dh/2), libm
 * sin/cos as on a non-Apple host (llama.h:5633-5636). */
TMO_API void tmo_rope_head(float* r, int dh, int pos, float theta) {
    int half = dh / 2;
    for (int j = 0; j < half; j++) {
        float inv = powf(theta, -2.0f * (float)j / (float)dh);
        float phase = (float)pos * inv;
        float s = sinf(phase), c = cosf(phase);
        float a = r[j], b = r[j + half];
        r[j] = a * c - b * s;
        r[j + half] = b * c + a * s;
    }
}

/* The (cos, sin) angle table a GPU backend builds on the host, metal.h:3926-3941:
 * entry [p*half + j] = (cos, sin) of (float)p * pow(theta, -2j/dh). */
TMO_API void tmo_rope_table(float* cs, int dh, int npos, float theta) {
    int half = dh / 2;
    for (int j = 0; j < half; j++) {
        float inv = powf(theta, -2.0f * (float)j / (float)dh);
        for (int p = 0; p < npos; p++) {
            float ang = (float)p * inv;
            cs[2 * ((size_t)p * half + j)] = cosf(ang);
            cs[2 * ((size_t)p * half + j) + 1] = sinf(ang);
        }
    }
}

/* One GQA group for one token, llama.h:4088-4111: S = scale * q K^T,
 * max-subtracted softmax per query head, out = S V. Kh/Vh are [allow][dh]. */
TMO_API void tmo_attn_group(const float* qg, const float* Kh, const float* Vh, float* out,
                            int REP, int dh, int allow, float scale) {
    float* S = (float*)malloc(sizeof(float) * (size_t)allow);
    for (int r = 0; r < REP; r++) {
        const float* q = qg + (size_t)r * dh;
        for (int s = 0; s < allow; s++) {
            float acc = 0.f;
            for (int k = 0; k < dh; k++) acc += q[k] * Kh[(size_t)s * dh + k];
            S[s] = scale * acc;
        }
        float m = -1e30f;
        for (int s = 0; s < allow; s++) m = fmaxf(m, S[s]);
        float z = 0.f;
        for (int s = 0; s < allow; s++) { S[s] = expf(S[s] - m); z += S[s]; }
        float inv = 1.f / z;
        for (int s = 0; s < allow; s++) S[s] *= inv;
        for (int k = 0; k < dh; k++) {
            float acc = 0.f;
            for (int s = 0; s < allow; s++) acc += S[s] * Vh[(size_t)s * dh + k];
            out[(size_t)r * dh + k] = acc;
        }
    }
    free(S);
}

/* SiLU(g) * u, llama.h:300 and 7109-7118. */
TMO_API void tmo_silu_mul(float* g, const float* u, int n) {
    for (int i = 0; i < n; i++) { float v = g[i]; g[i] = v / (1.f + expf(-v)) * u[i]; }
}

/* Greedy choice with the lowest-index tie rule (metal.h:2335). */
TMO_API unsigned tmo_argmax(const float* x, unsigned n) {
    unsigned best = 0; float bv = -INFINITY;
    for (unsigned i = 0; i < n; i++) if (x[i] > bv) { bv = x[i]; best = i; }
    return best;
}

/* ---- the decode chain -----------------------------------------------------------
 * Llama-style decoder, one token at a time, in the op order of the reference's
 * token encoder (llama.h:5818-5924): rmsnorm -> q|k|v GEMV -> rope(q), rope(k)
 * into the cache, v into the cache -> GQA attention over [0, pos] -> o GEMV ->
 * residual -> rmsnorm -> gate|up GEMV -> silu*up -> down GEMV -> residual;
 * final rmsnorm -> lm_head GEMV. KV caches are per layer [KVH][ctx][dh] fp32
 * (llama.h:5386-5410, rows written at 6797-6815). kv_half != 0 rounds K/V rows
 * to fp16 when they are written, as the reference GPU cache does by default
 * (metal.h:3968-3981). */
typedef struct {
    int L, D, H, KVH, dh, F, V, ctx;
    float theta, eps;
    int dt_proj, dt_head, dt_embed;        /* block dtypes */
    const void* embed;                      /* V x D */
    const void* head;                       /* V x D */
    const void* const* wq; const void* const* wk; const void* const* wv; const void* const* wo;
    const void* const* wgate; const void* const* wup; const void* const* wdown;
    const float* const* rms1; const float* const* rms2; const float* rmsf;
    float* kc; float* vc;                   /* L x [KVH][ctx][dh] */
    int kv_half;
    int threads;
    /* optional attention bias per layer (Qwen2-style; metal_llama.h:577-590, llama.h tok_bias_qkv): QD / KVD / KVD floats,
     * added to q, k, v before rope. NULL arrays: none. */
    const float* const* qb; const float* const* kb; const float* const* vb;
} tmo_model;

static void chain_gemv(const tmo_model* m, int dtype, const void* W, const float* x, float* y, int n_out, int n_in) {
    if (m->threads > 1) tmo_gemv_mt(dtype, W, x, y, n_out, n_in, m->threads);
    else tmo_gemv(dtype, W, x, y, n_out, n_in);
}

/* One forward at absolute position pos; logits has V floats. When taps != NULL it
 * receives, for layer tap_layer, the vectors at the op boundaries
 * [h(D) | qkv(QD+2KVD, after rope for q) | ao(QD) | x_after_attn(D) | h2(D) | act(F) | x_out(D)]. */
TMO_API int tmo_chain_step(const tmo_model* m, unsigned tok, int pos, float* logits, int tap_layer, float* taps) {
    int D = m->D, QD = m->H * m->dh, KVD = m->KVH * m->dh, F = m->F, REP = m->H / m->KVH;
    if (pos < 0 || pos >= m->ctx || (int)tok < 0 || (int)tok >= m->V) return 0;
    size_t be = (size_t)tmo_block_elems(m->dt_embed), bb = (size_t)tmo_block_bytes(m->dt_embed);
    float* x = (float*)malloc(sizeof(float) * (size_t)D);
    float* h = (float*)malloc(sizeof(float) * (size_t)D);
    float* qkv = (float*)malloc(sizeof(float) * (size_t)(QD + 2 * KVD));
    float* ao = (float*)malloc(sizeof(float) * (size_t)QD);
    float* t = (float*)malloc(sizeof(float) * (size_t)D);
    float* gu = (float*)malloc(sizeof(float) * (size_t)(2 * F));
    float* Kf = (float*)malloc(sizeof(float) * (size_t)(pos + 1) * m->dh);
    (void)Kf;
    tmo_dequant(m->dt_embed, (const uint8_t*)m->embed + (size_t)tok * ((size_t)D / be) * bb, x, (size_t)D);
    float scale = 1.f / sqrtf((float)m->dh);
    size_t lstride = (size_t)m->KVH * m->ctx * m->dh;
    for (int l = 0; l < m->L; l++) {
        float* kc = m->kc + (size_t)l * lstride;
        float* vc = m->vc + (size_t)l * lstride;
        tmo_rmsnorm(x, m->rms1[l], h, D, m->eps);
        chain_gemv(m, m->dt_proj, m->wq[l], h, qkv, QD, D);
        chain_gemv(m, m->dt_proj, m->wk[l], h, qkv + QD, KVD, D);
        chain_gemv(m, m->dt_proj, m->wv[l], h, qkv + QD + KVD, KVD, D);
        if (m->qb && m->kb && m->vb && m->qb[l]) {
            for (int i = 0; i < QD; i++) qkv[i] += m->qb[l][i];
            for (int i = 0; i < KVD; i++) { qkv[QD + i] += m->kb[l][i]; qkv[QD + KVD + i] += m->vb[l][i]; }
        }
        for (int hd = 0; hd < m->H; hd++) tmo_rope_head(qkv + (size_t)hd * m->dh, m->dh, pos, m->theta);
        for (int kv = 0; kv < m->KVH; kv++) {
            float* kr = qkv + QD + (size_t)kv * m->dh;
            tmo_rope_head(kr, m->dh, pos, m->theta);
            float* kd = kc + ((size_t)kv * m->ctx + pos) * m->dh;
            float* vd = vc + ((size_t)kv * m->ctx + pos) * m->dh;
            const float* vr = qkv + QD + KVD + (size_t)kv * m->dh;
            for (int i = 0; i < m->dh; i++) {
                kd[i] = m->kv_half ? tmo_fp16_to_fp32(tmo_fp32_to_fp16(kr[i])) : kr[i];
                vd[i] = m->kv_half ? tmo_fp16_to_fp32(tmo_fp32_to_fp16(vr[i])) : vr[i];
            }
        }
        if (taps && l == tap_layer) { memcpy(taps, h, 4 * (size_t)D); memcpy(taps + D, qkv, 4 * (size_t)(QD + 2 * KVD)); }
        for (int kv = 0; kv < m->KVH; kv++)
            tmo_attn_group(qkv + (size_t)kv * REP * m->dh, kc + (size_t)kv * m->ctx * m->dh,
                           vc + (size_t)kv * m->ctx * m->dh, ao + (size_t)kv * REP * m->dh,
                           REP, m->dh, pos + 1, scale);
        chain_gemv(m, m->dt_proj, m->wo[l], ao, t, D, QD);
        for (int i = 0; i < D; i++) x[i] += t[i];
        if (taps && l == tap_layer) {
            float* p = taps + D + QD + 2 * KVD;
            memcpy(p, ao, 4 * (size_t)QD); memcpy(p + QD, x, 4 * (size_t)D);
        }
        tmo_rmsnorm(x, m->rms2[l], h, D, m->eps);
        chain_gemv(m, m->dt_proj, m->wgate[l], h, gu, F, D);
        chain_gemv(m, m->dt_proj, m->wup[l], h, gu + F, F, D);
        tmo_silu_mul(gu, gu + F, F);
        chain_gemv(m, m->dt_proj, m->wdown[l], gu, t, D, F);
        for (int i = 0; i < D; i++) x[i] += t[i];
        if (taps && l == tap_layer) {
            float* p = taps + D + QD + 2 * KVD + QD + D;
            memcpy(p, h, 4 * (size_t)D); memcpy(p + D, gu, 4 * (size_t)F); memcpy(p + D + F, x, 4 * (size_t)D);
        }
    }
    tmo_rmsnorm(x, m->rmsf, h, D, m->eps);
    chain_gemv(m, m->dt_head, m->head, h, logits, m->V, D);
    free(x); free(h); free(qkv); free(ao); free(t); free(gu); free(Kf);
    return 1;
}
