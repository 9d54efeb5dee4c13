/* include/llama_gpu_api.h — plain-C contract of the GPU prefill layer stack.
 *
 * The declarations of the reference's tensormark/llama_gpu_api.h:9-30 (same structs, same parameter lists, same
 * return conventions), implemented for B200 in tensormark_b200/csrc/llama_stack.cu. Every entry exists under its
 * tm_cuda_* name and under the reference's tm_metal_* name, so a caller written against the reference links
 * without change (the reference's engine declares these weak and tests them for null, tensormark/llama.h:35-152).
 *
 * What the stack does (tensormark/metal_llama.h:521-719 encode_layer, 727-775 create, 897-998 prefill and the
 * begin / wait_layer / end form): for a batch of T >= 2 tokens at positions pos0 .. pos0+T-1 it runs, per layer,
 * rmsnorm -> q/k/v GEMMs (-> attention bias) -> rope(q, k) -> K/V rows appended to the caches -> causal GQA
 * attention over [0, pos] -> o GEMM + residual -> rmsnorm -> gate/up GEMMs -> silu*up -> down GEMM + residual, on
 * the T x D residual stream x (fp32, in/out).
 *
 * Ownership, as in the reference: every pointer is caller-owned HOST memory. Weight pointers lie inside
 * [map_base, map_base + map_size) when a mapping is named (it is made resident on the device once and shared with
 * the decode lane's registrations); map_base == NULL registers each tensor by itself. kc / vc are the caller's
 * fp32 caches [KVH][ctx][dh]: the reference's GPU writes into them through unified memory; here the stack keeps
 * device copies and writes the rows it computes back into the caller's arrays (prefill: before it returns;
 * begin/wait_layer: layer l's rows are there when wait_layer(l) returns 1). Rows [0, pos0) are read from the
 * caller's arrays at the start of every call with pos0 > 0, as unified memory would show them.
 * Not in the reference: a layer whose kc and vc are both NULL keeps its rows on the device only (nothing is copied
 * either way; a call with pos0 > 0 continues from the rows earlier calls left there); tm_cuda_llama_kv_to_slots
 * hands them to the decode lane.
 * Constraints: dh even (64 or 128 for the attention kernel), H % KVH == 0, T >= 2, pos0 + T <= ctx; blocks are Q4_0
 * unless the *_create_dt form names another block format.
 * Errors: create returns NULL, the int entries return 0, and tm_cuda_last_error() names the reason. */
#ifndef TM_LLAMA_GPU_API_H
#define TM_LLAMA_GPU_API_H
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif
typedef struct tm_llama_gpu_layer {
    const void *q, *k, *v, *o, *gate, *up, *down;   /* block streams (inside the mapping when one is named) */
    const float* rms1; const float* rms2;           /* D floats each */
    const float* q_bias; const float* k_bias; const float* v_bias;  /* attention bias (QD/KVD/KVD); may be null */
    float* kc; float* vc;                            /* [KVH][ctx][dh] */
} tm_llama_gpu_layer;
typedef struct tm_llama_gpu_desc {
    int L, D, H, KVH, dh, F, ctx;
    float theta, eps;
    const void* map_base; size_t map_size;
    const tm_llama_gpu_layer* layers;
} tm_llama_gpu_desc;

/* llama_gpu_api.h:21-30 */
void* tm_cuda_llama_create(const tm_llama_gpu_desc* d);
int tm_cuda_llama_prefill(void* h, float* x, int T, int pos0);                 /* x: T x D in/out; 1 on success */
int tm_cuda_llama_prefill_begin(void* h, const float* x, int T, int pos0);     /* enqueues every layer, x is not written back */
int tm_cuda_llama_prefill_wait_layer(int l);                                   /* layer l's K/V rows are in the caller's arrays */
int tm_cuda_llama_prefill_end(void);
double tm_cuda_llama_prefill_gpu_ms(void);                                     /* GPU time of the last finished prefill */
/* Not in the reference: the batch buffers for prompts of up to T tokens now instead of inside the first prefill. */
int tm_cuda_llama_reserve(void* h, int T);
/* Not in the reference: prefill_begin whose residual stream is gathered on the device - row toks[t] of the
 * block-quantized embedding table registered with the decode lane as (wid, woff), `vocab` rows of D values in block
 * format `dtype`, dequantized exactly - instead of uploaded from host rows. */
int tm_cuda_llama_prefill_begin_tokens(void* h, const int* toks, int T, int pos0, int wid, unsigned long long woff, int vocab, unsigned dtype);
void tm_cuda_llama_destroy(void* h);

void* tm_metal_llama_create(const tm_llama_gpu_desc* d);
int tm_metal_llama_prefill(void* h, float* x, int T, int pos0);
int tm_metal_llama_prefill_begin(void* h, const float* x, int T, int pos0);
int tm_metal_llama_prefill_wait_layer(int l);
int tm_metal_llama_prefill_end(void);
double tm_metal_llama_prefill_gpu_ms(void);
void tm_metal_llama_destroy(void* h);

/* No counterpart in the reference (its stack is Q4_0-only, tensormark/llama.h:3960, 4463): the same stack over
 * another block format of the container (tensormark/tmq.h:48-60: 0 Q8_0, 1 Q4_0, 4 Q4_1, 5 Q5_K, 6 Q6_K, 8 Q4_K). */
void* tm_cuda_llama_create_dt(const tm_llama_gpu_desc* d, unsigned dtype);
/* No counterpart in the reference, whose decode lane re-uploads the prefilled rows from unified memory
 * (tensormark/llama.h:5738-5744): rows [pos0, pos0 + T) of layer l's device K/V caches into two K/V slots of the
 * decode lane (include/cuda_shim.h, tm_cuda_tok_kv_reserve), converted to the lane's cache precision, without a
 * trip through host memory. Enqueued on the lane's stream; 1 on success. */
int tm_cuda_llama_kv_to_slots(void* h, int l, int kcslot, int vcslot, int pos0, int T);
#ifdef __cplusplus
}
#endif
#endif /* TM_LLAMA_GPU_API_H */
