// glue.h — launchers of the decode-chain glue kernels (glue.cu).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "common.cuh"

namespace tmc {

bool launch_rmsnorm(const float* x, const float* w, float* out, unsigned D, float eps, cudaStream_t st);
bool launch_add(float* a, const float* b, unsigned n, cudaStream_t st);
bool launch_silu_mul(float* g, const float* u, unsigned n, cudaStream_t st);
bool launch_bias(float* y, const float* bias, unsigned n, cudaStream_t st);
bool launch_copy_bytes(const uint8_t* src, uint8_t* dst, unsigned n, cudaStream_t st);
// tbl: (cos, sin) float pairs, entry [pos * dh/2 + j]; tbl_entries = number of pairs
bool launch_rope(float* q, unsigned heads, unsigned dh, int pos, const float* tbl, unsigned tbl_entries, cudaStream_t st);
bool launch_rope_k_cache(const float* ksrc, void* cache, bool half_cache, unsigned KVH, unsigned dh, unsigned ctx, int pos,
                         const float* tbl, unsigned tbl_entries, cudaStream_t st);
bool launch_v_cache(const float* v, void* cache, bool half_cache, unsigned KVH, unsigned dh, unsigned ctx, int pos, cudaStream_t st);
bool launch_f32_to_half(const float* src, void* dst, size_t n, cudaStream_t st);
bool launch_half_to_f32(const void* src, float* dst, size_t n, cudaStream_t st);
// state (optional, device): chain state {position, token index}; when given, position and index come from it
bool launch_embed_row(const unsigned* tok, unsigned idx, const uint8_t* W, float* x, unsigned D, unsigned dtype, cudaStream_t st,
                      const int* state = nullptr);
// scratch: two zero-initialised 64-bit words owned by the caller, re-armed by the kernel
bool launch_choose_shard(const float* x, unsigned* out, unsigned lo, unsigned n, float inv_temp, unsigned seed, bool sample,
                         unsigned long long* scratch, unsigned long long* keys, cudaStream_t st, const int* state, const Exchange& xc);
bool launch_choose(const float* x, unsigned* out, unsigned n, unsigned idx, float inv_temp, unsigned seed, bool sample,
                   unsigned long long* scratch, cudaStream_t st, const int* state = nullptr, const Exchange* xchg = nullptr);

struct AttnPlan {
    unsigned nsplit;        // 0: the scratch cannot hold even one split
    unsigned chunk;         // positions per split
    size_t part_floats;     // floats of partial outputs; the (max, sum) stats follow them
};
// scratch_bytes: size of the buffer that will receive partials and stats.
AttnPlan plan_attention(unsigned H, unsigned KVH, unsigned dh, unsigned ctx, unsigned allow, size_t scratch_bytes);
// The same rule for a caller that names the SM count itself (a scratch_bytes of 1 << 40 means: no limit from the buffer).
AttnPlan plan_attention_sms(unsigned sms, unsigned H, unsigned KVH, unsigned dh, unsigned ctx, unsigned allow, size_t scratch_bytes);
bool launch_attention(const float* q, const void* kc, const void* vc, bool half_cache, float* scratch, float* out,
                      unsigned H, unsigned KVH, unsigned dh, unsigned ctx, unsigned allow, float scale, unsigned REP,
                      const AttnPlan& pl, cudaStream_t st, const int* state = nullptr);
bool launch_qkv_post(float* qkv, void* kc, void* vc, bool half_cache, unsigned H, unsigned KVH, unsigned dh, unsigned ctx,
                     const float* tbl, unsigned tbl_entries, const int* state, cudaStream_t st);
bool launch_advance(int* state, cudaStream_t st);
// One launch for rope(q), rope(k) -> cache, v -> cache, split-K attention over [0, position] and the merge
// (attn_fused.cu). qkv = [q | k | v] of the current token, un-rotated; scratch as for launch_attention.
unsigned attn_fused_splits(unsigned H, unsigned KVH, unsigned dh, unsigned ctx, size_t scratch_bytes);
bool launch_attn_fused(const float* qkv, void* kc, void* vc, bool half_cache, float* scratch, size_t scratch_bytes, float* out,
                       unsigned H, unsigned KVH, unsigned dh, unsigned ctx, float scale, const float* tbl, unsigned tbl_entries,
                       const int* state, cudaStream_t st);

}  // namespace tmc
