/* include/cuda_shim.h — C ABI of the B200 backend for TensorMark's quantized-weight
 * matmul path.
 *
 * This is the drop-in boundary: the library (libtm_cuda.so) exports, for every
 * entry point of the reference's Metal shim that lies on the quantized matmul /
 * decode-chain path, a `tm_cuda_*` function with the same parameter list and the
 * same meaning, plus a `tm_metal_*` alias so a caller written against the
 * reference's weak-import declarations (tensormark/llama.h:35-152) links without
 * change. Citations name the reference interface each entry replaces.
 *
 * Conventions kept from the reference:
 *   - `bool` entries return false on any failure and bump tm_cuda_fallback_count()
 *     (tensormark/metal.h:46-59, "a counter, not a print"). There is no CPU path
 *     behind a false: the caller decides what to do.
 *   - `void` token-lane encoders cannot report; where the reference throws a C++
 *     exception across the C boundary (e.g. metal.h:3526, 4160) this library
 *     latches a sticky error that makes the next tok_end / tok_flush /
 *     tok_wait_pending return false. tm_cuda_last_error() names it.
 *   - dtype codes are the container's (tensormark/tmq.h:48-60):
 *     0 Q8_0, 1 Q4_0, 3 F16, 4 Q4_1, 5 Q5_K, 6 Q6_K, 8 Q4_K, 9 GGUF-native Q4_0, 10 BF16.
 *   - Host-pointer entries are blocking and, like the reference's function-local
 *     caches, not thread-safe: one caller thread per process.
 *
 * Entries ending in `_dev` take DEVICE pointers and a stream (a cudaStream_t
 * passed as void*; NULL = the legacy default stream) and never synchronize. They
 * are what the token lane launches internally, exported so a resident caller (or
 * a benchmark) can time the kernels without host copies.
 */
#ifndef TM_CUDA_SHIM_H
#define TM_CUDA_SHIM_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TM_DT_Q8_0 0u
#define TM_DT_Q4_0 1u
#define TM_DT_F16  3u
#define TM_DT_Q4_1 4u
#define TM_DT_Q5_K 5u
#define TM_DT_Q6_K 6u
#define TM_DT_Q4_K 8u
#define TM_DT_GGUF_Q4_0 9u   /* GGUF's own Q4_0: split nibbles (tensormark/tmq.h:58, llama.h:4588-4597) */
#define TM_DT_BF16 10u

/* ---- library state ------------------------------------------------------- */
/* Select the device for this process and create the lane stream. Called lazily
 * by every other entry (the reference's ensure_init, metal.h:73-91). */
bool tm_cuda_init(int device);
/* Message of the most recent failure, "" when none. */
const char* tm_cuda_last_error(void);
/* Number of entries that returned false so far (metal.h:46-59 fallback_count). */
unsigned long long tm_cuda_fallback_count(void);
/* Number of kernels of this library launched so far in this process. */
unsigned long long tm_cuda_launch_count(void);
/* Kernel timeline, for tuning (no counterpart in the reference). With TM_CUDA_TRACE=1 in the
 * environment at tm_cuda_init, CTA 0 of every GEMV records six 64-bit words: %globaltimer (ns) at its
 * start, after the wait for the preceding kernel, after x is staged, at its end; then (N << 32 | K) and
 * (dtype | x_op << 8 | warps << 16 | rows-per-item << 24). The fused chain attention records, for its
 * CTA (0, 0): start, after the wait, after its prologue, after the split handoff, after its tiles, and
 * the handoff time again (words 4 and 5 are then timestamps). tm_cuda_trace_read synchronises the lane,
 * copies up to cap_launches records (in launch-start order) and clears the log. Returns the count; 0
 * when tracing is off. At most 8192 launches are kept between reads. */
size_t tm_cuda_trace_read(unsigned long long* out, size_t cap_launches);
/* Number of multiprocessors of the selected device. */
int tm_cuda_sm_count(void);
/* Limit, in milliseconds, of every device-side wait on another GPU (the peer gather's counters). Default 2000, or
 * TM_CUDA_WAIT_LIMIT_MS at tm_cuda_init. A wait that runs out does not hang or fault: the kernel goes on, the next
 * synchronising entry (tok_flush / tok_end / tok_wait_pending) returns false and tm_cuda_last_error() says that a
 * kernel gave up on a bounded wait; later waits of the same token stream return at once until then. The analogue
 * of the reference's 30 s deadline on its GPU/CPU hand-off (metal_llama.h:856-876). ms == 0 only reads.
 * Returns the previous limit. Applies to launches encoded afterwards. */
unsigned tm_cuda_set_wait_limit_ms(unsigned ms);

/* ---- per-tensor projection, host pointers -------------------------------- */
/* y[N] = W[N x K] . x[K], W Q4_0 blocks. Weights are cached on the device keyed
 * by (pointer, bytes); x and y are copied per call. K % 32 != 0 -> false.
 * Replaces tm_metal_q4_gemv (metal_shim.mm:17-20, metal.h:2058-2127); bound to
 * tmllama::Q4Gemv (q4_projection_backend.h:7-8). */
bool tm_cuda_q4_gemv(const float* x, const void* Wq, float* y, unsigned N, unsigned K);
/* C[M x N] = A[M x K] . W^T, W Q4_0. Replaces tm_metal_sgemm_q4
 * (metal_shim.mm:6-9, metal.h:1981-2052); bound to tmllama::Q4Gemm. */
bool tm_cuda_sgemm_q4(const float* A, const void* Wq, float* C, unsigned M, unsigned N, unsigned K);
/* Fused multi-tensor prefill: C is M x sum(Ns) row-major, part p occupying the
 * columns after parts 0..p-1. Replaces tm_metal_q4_prefill (metal_shim.mm:11-15,
 * metal.h:2133-2235). */
bool tm_cuda_q4_prefill(const float* A, const void* const* Wqs, const unsigned* Ns, unsigned nparts,
                        float* C, unsigned M, unsigned K);
/* dtype-carrying forms of the three above (the reference's per-call entries are
 * Q4_0-only; its token lane carries the dtype, metal_shim.mm:84-89). */
bool tm_cuda_gemv_q(const float* x, const void* W, float* y, unsigned N, unsigned K, unsigned dtype);
bool tm_cuda_sgemm_q(const float* A, const void* W, float* C, unsigned M, unsigned N, unsigned K, unsigned dtype);
/* out[N x K] fp32 = dequantized W; bit-exact against tmq::dequantize_row_*
 * (quant.h:194-200, 267-277, 304-330, 338-365, 397-408). The fp32 form of
 * q4_dequant_f32 (metal.h:1516-1562), for every block dtype. */
bool tm_cuda_dequant(const void* W, float* out, unsigned N, unsigned K, unsigned dtype);
/* Drop every device copy of weights this library holds: the caches of the host-pointer entries, the
 * token lane's registrations (their handles become invalid; handle ids are not reused), the cached norm
 * weights, and every lane graph. Copies are keyed by HOST address, as in the reference, so a caller
 * that frees a tensor and may get the same address back for another one calls this in between. */
void tm_cuda_release_weights(void);

/* ---- device-pointer kernels ---------------------------------------------- */
/* Bytes of an N x K tensor of `dtype`; 0 when K is not whole blocks (tmq.h:124-133). */
size_t tm_cuda_weight_bytes(unsigned dtype, size_t N, size_t K);
/* y = W x. W must be 16-byte aligned. (metal.h:3457-3480 tok_gemv, 3647-3669 tok_gemv_kq; dtype 3 / 10: plain fp16 /
 * bf16 rows, metal.h:575-613 f16_gemv_coop and 3693-3721 tok_gemv_h) */
bool tm_cuda_gemv_q_dev(const float* x, const void* W, float* y, unsigned N, unsigned K, unsigned dtype, void* stream);
/* nblocks Q4_0 blocks in GGUF's split nibble order, rewritten in place in the container's interleaved order (what the
 * reference's converter does on the host, convert_gguf.cpp:124-135): same scale, same codes, bit-identical weights. */
bool tm_cuda_q4_0_from_gguf_dev(void* blocks, size_t nblocks, void* stream);
/* Segmented GEMV: N total rows over nseg segments; segment s covers seg_rows[s]
 * rows whose blocks start seg_woff[s] bytes after W. One launch; every row is
 * computed exactly as the unsegmented kernel computes it. nseg <= 16.
 * (metal.h:3519-3556 tok_gemv_seg, 3585-3616 tok_gemv_seg_dt) */
bool tm_cuda_gemv_seg_dev(const float* x, const void* W, float* y, unsigned N, unsigned K, unsigned dtype,
                          const uint64_t* seg_woff, const unsigned* seg_rows, unsigned nseg, void* stream);
bool tm_cuda_dequant_dev(const void* W, float* out, unsigned N, unsigned K, unsigned dtype, void* stream);
/* C[M x N] = A[M x K] . W^T on the tensor cores. `workspace` is device scratch of
 * at least tm_cuda_sgemm_q_workspace(M, N, K, dtype) bytes, 256-byte aligned. */
size_t tm_cuda_sgemm_q_workspace(unsigned M, unsigned N, unsigned K, unsigned dtype);
bool tm_cuda_sgemm_q_dev(const float* A, const void* W, float* C, unsigned M, unsigned N, unsigned K,
                         unsigned dtype, void* workspace, size_t workspace_bytes, void* stream);

/* Decode glue on device pointers (the kernels behind the token lane). */
bool tm_cuda_rmsnorm_dev(const float* x, const float* w, float* out, unsigned D, float eps, void* stream);
bool tm_cuda_add_dev(float* a, const float* b, unsigned n, void* stream);
bool tm_cuda_silu_mul_dev(float* g, const float* u, unsigned n, void* stream);
bool tm_cuda_argmax_dev(const float* x, unsigned* out, unsigned n, void* stream);
/* GQA split-K decode attention for one token (metal.h:2739-2859, host side 4153-4222): q is
 * [H][dh] fp32, kc/vc are [KVH][ctx][dh] caches (half when kv_half != 0, else fp32), positions
 * [0, allow) are attended, out is [H][dh]. `scratch` receives the per-split partial outputs and
 * softmax statistics; it must hold at least tm_cuda_attn_decode_scratch(...) bytes. */
size_t tm_cuda_attn_decode_scratch(unsigned H, unsigned KVH, unsigned dh, unsigned ctx, unsigned allow);
bool tm_cuda_attn_decode_dev(const float* q, const void* kc, const void* vc, float* scratch, size_t scratch_bytes,
                             float* out, unsigned H, unsigned KVH, unsigned dh, unsigned ctx, unsigned allow,
                             float scale, int kv_half, void* stream);
/* The same attention for callers that cannot allocate device memory. It has no counterpart in
 * the reference; it exists for hosts that have given all free device memory to their own pool
 * (so a cudaMalloc for scratch would fail) or that cannot afford cudaMalloc's device-wide
 * synchronisation on their token path. The split-K scratch is a static array inside the library,
 * TM_CUDA_ATTN_STATIC_SCRATCH_BYTES per GPU, held from library load to process exit; the call
 * performs no cudaMalloc/cudaFree and uses no allocating routine. Shapes whose scratch would not
 * fit are refused (false, tm_cuda_last_error() says how many bytes were needed). The first call on
 * a device looks up the array's device address: make that call before any stream capture starts.
 * Every call shares the one array, so calls that may overlap on the GPU (different streams,
 * different threads) race with each other; within one stream, back-to-back calls are safe. */
#define TM_CUDA_ATTN_STATIC_SCRATCH_BYTES (512u * 1024u)
bool tm_cuda_attn_decode_static_dev(const float* q, const void* kc, const void* vc, float* out, unsigned H,
                                    unsigned KVH, unsigned dh, unsigned ctx, unsigned allow, float scale,
                                    int kv_half, void* stream);

/* ---- token lane (metal_shim.mm:22-152) ----------------------------------- */
/* Slots are backend-owned grow-only device buffers addressed by small integers
 * (metal.h:2262-2281). A slot may not grow between tok_begin and the matching
 * end (metal.h:3135-3140): reserve packed outputs first. */
bool tm_cuda_tok_begin(void);                                   /* metal.h:3074-3089 */
bool tm_cuda_tok_flush(void);                                   /* metal.h:3109-3121 */
bool tm_cuda_tok_end(int outslot, float* dst, unsigned n);      /* metal.h:3122-3127 */
bool tm_cuda_tok_end_async(void);                               /* metal.h:3152-3158 */
bool tm_cuda_tok_wait_pending(void);                            /* metal.h:3161-3190 */
bool tm_cuda_tok_reserve(int slot, size_t bytes);               /* metal.h:3135-3140 */
bool tm_cuda_tok_upload(int slot, size_t byte_off, const void* src, size_t bytes);   /* metal.h:3128-3134 */
bool tm_cuda_tok_download(int slot, size_t byte_off, void* dst, size_t bytes);       /* metal.h:3141-3147 */
/* K/V cache slots; offsets and counts are in ELEMENTS, the element type is half
 * unless TM_CUDA_KV_HALF=0 (metal.h:3968-4014). */
bool tm_cuda_tok_kv_reserve(int slot, size_t n);
bool tm_cuda_tok_kv_upload(int slot, size_t elem_off, const float* src, size_t n);
bool tm_cuda_tok_kv_download(int slot, size_t elem_off, float* dst, size_t n);
/* Register a weight tensor; returns a handle >= 1000 (or -1) and the byte offset
 * of the tensor inside the handle's buffer. With zero_copy != 0 the whole mapping
 * [map_base, map_base+map_size) is made resident once and every tensor inside it
 * shares one handle, as the reference's NoCopy buffer does (metal.h:3282-3337);
 * "zero copy" on a discrete GPU is one aligned host-to-device copy of the mapping.
 * The reference declares woff_out as a C++ reference; a pointer is the same ABI. */
int tm_cuda_tok_wbuf(const void* tensor_ptr, size_t bytes, const void* map_base, size_t map_size,
                     int zero_copy, uint64_t* woff_out);
/* n tensors into one device buffer at 256-byte aligned offsets, one handle for all (no counterpart in the
 * reference, whose unified memory aliases the file mapping): for tensors that lie at arbitrary offsets of a
 * container file but must be row-aligned on the device and share a handle for segmented GEMVs. Afterwards
 * tm_cuda_tok_wbuf(tensor_ptrs[i], ...) returns this handle and woff_out[i]. Returns the handle or -1. */
int tm_cuda_tok_wbuf_pack(const void* const* tensor_ptrs, const size_t* bytes, unsigned n, uint64_t* woff_out);
bool tm_cuda_tok_probe_copy(int srcslot, size_t src_off, int dstslot, unsigned n);   /* metal.h:3338-3351 */
void tm_cuda_tok_gemv(int xslot, int wid, uint64_t woff, int yslot, size_t yoff, unsigned N, unsigned K);
bool tm_cuda_tok_gemv_seg_supported(unsigned dtype);             /* metal.h:3513-3518 */
void tm_cuda_tok_gemv_seg(int xslot, int wid, int yslot, size_t yoff, unsigned N, unsigned K,
                          const uint64_t* seg_woff, const unsigned* seg_rows, unsigned nseg);
void tm_cuda_tok_gemv_seg_dt(int xslot, int wid, int yslot, size_t yoff, unsigned N, unsigned K, unsigned dtype,
                             const uint64_t* seg_woff, const unsigned* seg_rows, unsigned nseg);
/* dtype in {0, 1, 4, 5, 6}: the reference has no Q8_0 GPU GEMV (llama.h:1264-1268);
 * this backend serves it through the same entry. */
void tm_cuda_tok_gemv_kq(int xslot, int wid, uint64_t woff, int yslot, size_t yoff, unsigned N, unsigned K,
                         unsigned dtype);
void tm_cuda_tok_embed_q4(int tokslot, unsigned idx, int wid, uint64_t woff, int xslot, unsigned D);  /* metal.h:3227-3240 */
void tm_cuda_tok_embed_kq(int tokslot, unsigned idx, int wid, uint64_t woff, int xslot, unsigned D, unsigned dtype);
void tm_cuda_tok_gemv_h(int xslot, int wid, uint64_t woff, int yslot, size_t yoff, unsigned N, unsigned K);   /* F16 tensor; metal.h:3693-3721 */
void tm_cuda_tok_embed_h(int tokslot, unsigned idx, int wid, uint64_t woff, int xslot, unsigned D);           /* metal.h:3260-3271 */
/* The same reorder for a registered weight range (blocking); afterwards the range is container Q4_0 (dtype 1). */
bool tm_cuda_tok_wbuf_q4_from_gguf(int wid, uint64_t woff, size_t nblocks);
void tm_cuda_tok_bias_qkv(int yslot, int biasslot, size_t bias_off, unsigned N);     /* metal.h:3672-3688 */
void tm_cuda_tok_rmsnorm(int xslot, const void* w, int outslot, unsigned D, float eps);  /* metal.h:3722-3746 */
void tm_cuda_tok_add(int a, int b, unsigned n);                                      /* metal.h:3747-3754 */
void tm_cuda_tok_silu_mul(int g, size_t goff, int u, size_t uoff, unsigned n);       /* metal.h:3755-3765 */
void tm_cuda_tok_rope_q(int qslot, unsigned H, unsigned dh, int pos, float theta);   /* metal.h:3950-3967 */
void tm_cuda_tok_rope_k_cache(int ksrcslot, size_t ksrc_off, int cacheslot, unsigned KVH, unsigned dh,
                              unsigned ctx, int pos, float theta);                   /* metal.h:4015-4034 */
void tm_cuda_tok_v_cache(int vsrcslot, size_t vsrc_off, int cacheslot, unsigned KVH, unsigned dh,
                         unsigned ctx, int pos);                                     /* metal.h:4035-4049 */
void tm_cuda_tok_attn(int qslot, int kcslot, int vcslot, int probslot, int outslot, unsigned QD, unsigned H,
                      unsigned KVH, unsigned dh, unsigned ctx, int allow, float scale, unsigned REP);  /* metal.h:4153-4275 */
void tm_cuda_tok_argmax(int xslot, int tokslot, unsigned idx, unsigned n);           /* metal.h:3191-3200 */
void tm_cuda_tok_sample(int xslot, int tokslot, unsigned idx, unsigned n, float inv_temp, unsigned seed);  /* metal.h:3201-3212 */
unsigned tm_cuda_tok_peek(int tokslot, unsigned idx);                                /* metal.h:3216-3226 */
/* ---- chain forms (no counterpart in the reference's shim; they serve its greedy chain,
 * llama.h:6047-6165, without one host round trip per token) --------------------------------
 * A "chain state" is two ints in a slot: {position, token index}. The entries below read it on
 * the device, so ONE captured graph of a token's launches is replayed for every token:
 * embed(tok[index]) -> layers at `position` -> argmax -> tok[index+1] -> advance. */
/* GEMV with optional fusions: x_op 0 = plain, 1 = RMSNorm(x; norm_w, eps) applied while x is
 * staged, 2 = silu(x) * x2 (x2 at x2slot/x2off); accumulate != 0 adds the result to y (residual).
 * Segments as tok_gemv_seg_dt. */
void tm_cuda_tok_gemv_fused(int xslot, size_t xoff, int x_op, int x2slot, size_t x2off, const void* norm_w, float eps,
                            int wid, int yslot, size_t yoff, unsigned N, unsigned K, unsigned dtype,
                            const uint64_t* seg_woff, const unsigned* seg_rows, unsigned nseg, int accumulate);
/* rope(q) in place + rope(k) -> K cache + v -> V cache for the packed q|k|v slot, one launch. */
void tm_cuda_tok_qkv_post_at(int qkvslot, int kcslot, int vcslot, unsigned H, unsigned KVH, unsigned dh, unsigned ctx,
                             float theta, int stateslot);
void tm_cuda_tok_attn_at(int qslot, int kcslot, int vcslot, int probslot, int outslot, unsigned QD, unsigned H,
                         unsigned KVH, unsigned dh, unsigned ctx, float scale, unsigned REP, int stateslot);
/* tok[index + 1] = argmax(x[0..n)); the token slot holds max_tokens entries. */
/* tok_qkv_post_at and tok_attn_at as ONE launch: rope(q), rope(k) -> K cache, v -> V cache, attention
 * over [0, position] and the merge of its splits. qkvslot holds the token's un-rotated [q | k | v]; q is
 * not written back. probslot is scratch: (dh + 2) * H * 4 bytes per split, as many splits as fit up to
 * one CTA per SM. (metal.h:3950-4030, 4153-4222 in one dispatch.) */
/* The merge of the splits uses one counter per K/V head that is shared by every call of this entry in the process:
 * calls must not overlap on the GPU (the lane issues them on its one stream, which orders them). */
void tm_cuda_tok_attn_fused_at(int qkvslot, int kcslot, int vcslot, int probslot, int outslot, unsigned H, unsigned KVH,
                               unsigned dh, unsigned ctx, float scale, float theta, int stateslot);
void tm_cuda_tok_argmax_at(int xslot, int tokslot, unsigned n, unsigned max_tokens, int stateslot);
/* Chain form of tok_sample (Gumbel-max, metal.h:2349-2379): the noise is the reference's hash of (seed, token
 * index, vocabulary index), the token index coming from the chain state; inv_temp <= 0 is the plain argmax.
 * wait_site >= 0: wait for that gather first (row-sharded models), -1 otherwise. */
void tm_cuda_tok_sample_at(int xslot, int tokslot, unsigned n, unsigned max_tokens, float inv_temp, unsigned seed, int stateslot,
                           int wait_site);
/* x = row tok[index] of the embedding table. */
void tm_cuda_tok_embed_at(int tokslot, int wid, uint64_t woff, int xslot, unsigned D, unsigned dtype, unsigned max_tokens,
                          int stateslot);
void tm_cuda_tok_advance(int stateslot);                         /* position, index and exchange epoch += 1 (a state is 4 ints) */
/* Capture the launches encoded between begin and end into a CUDA graph (returns its id, -1 on
 * failure) and replay it. Slots, weight handles and norm weights must exist before the capture. */
bool tm_cuda_tok_graph_begin(void);
int tm_cuda_tok_graph_end(void);
bool tm_cuda_tok_graph_launch(int id, unsigned times);
void tm_cuda_tok_graph_destroy(int id);                         /* id < 0: every graph of the lane */

/* ---- row-sharded models: one process per GPU -------------------------------------------------
 * No counterpart in the reference, which runs on one GPU. A model whose FFN and LM-head rows are
 * spread over `world` GPUs gathers each sharded GEMV's output with tm_cuda_tok_all_gather, an
 * ncclAllGather on the lane's stream (captured into token graphs like any other op). NCCL is bound
 * at run time, on the first call that needs it. Rank 0 makes the id (tm_cuda_comm_id_bytes() bytes),
 * the caller carries it to the other ranks, and every rank calls tm_cuda_comm_init after
 * tm_cuda_init(device). tm_cuda_comm_destroy first destroys every graph of the lane. */
size_t tm_cuda_comm_id_bytes(void);
bool tm_cuda_comm_unique_id(void* out);
bool tm_cuda_comm_init(int rank, int world, const void* id_bytes);
int tm_cuda_comm_rank(void);
int tm_cuda_comm_world(void);
bool tm_cuda_comm_destroy(void);
/* dst[dst_off + r*count*4 ...) on every rank <- count floats at src[src_off] of rank r. In place when
 * src is this rank's slice of dst. Offsets and count*4 are multiples of 16. world == 1: a copy. */
void tm_cuda_tok_all_gather(int srcslot, size_t src_off, int dstslot, size_t dst_off, unsigned count);

/* The same gather without a collective kernel: each rank's arena is mapped into every peer (CUDA
 * IPC) and the GEMV that produces a shard stores each finished row into the peers' copies of the
 * output slot over NVLink as well as its own; every CTA then (barrier, one system-scope fence that orders
 * its rows before what follows) adds 1 to the rank's counter of the gather "site" on every peer with relaxed
 * reductions. The kernel that consumes the gathered vector waits until the other ranks' counters have reached
 * epoch * CTAs-of-the-producer (bounded: tm_cuda_set_wait_limit_ms, 2 s by default; then the status word
 * reports it and a sticky abort word stops every later wait on every rank) before it reads.
 * Set-up on every rank: tm_cuda_peer_arena -> exchange the handles -> tm_cuda_peer_open ->
 * tm_cuda_tok_reserve_shared for the gathered slots, in the same order on every rank. A site is an
 * index < 256 naming one gather per token; the chain state's fourth int is the token epoch
 * (tm_cuda_tok_advance increments it). Every rank must launch the same shapes. At most 8 ranks. */
size_t tm_cuda_peer_handle_bytes(void);
bool tm_cuda_peer_arena(size_t bytes, void* handle_out);
bool tm_cuda_peer_open(int rank, int world, const void* handles);
/* Rehearsal on ONE GPU (tests): every peer arena is this GPU's own arena, so pushes land locally and the other
 * ranks' counters never advance; a kernel that waits for them runs into the wait limit. */
bool tm_cuda_peer_open_loopback(int rank, int world);
/* Rehearsals: advance rank `rank`'s counter of `site` in this rank's arena by `count` (stream-ordered), as that
 * rank's pushes would. */
bool tm_cuda_peer_bump(int site, int rank, unsigned count);
int tm_cuda_peer_world(void);
int tm_cuda_peer_rank(void);
bool tm_cuda_peer_unmap(void);                                   /* then a barrier between the ranks, then: */
bool tm_cuda_peer_close(void);
bool tm_cuda_tok_reserve_shared(int slot, size_t bytes);
/* tm_cuda_tok_gemv_fused with (a) one output byte offset per segment (seg_yoff), (b) wait_site >= 0:
 * wait for that site's gather before reading x, (c) push_site >= 0: store the output rows into every
 * peer's copy of yslot (a shared slot) as well and signal that site. */
void tm_cuda_tok_gemv_xchg(int xslot, size_t xoff, int x_op, int x2slot, size_t x2off, const void* norm_w, float eps,
                           int wid, int yslot, const size_t* seg_yoff, unsigned N, unsigned K, unsigned dtype,
                           const uint64_t* seg_woff, const unsigned* seg_rows, unsigned nseg, int accumulate,
                           int wait_site, int push_site, int stateslot);
void tm_cuda_tok_argmax_xchg(int xslot, int tokslot, unsigned n, unsigned max_tokens, int stateslot, int wait_site);
/* The choice of a row-sharded LM head WITHOUT gathering the logits: this rank reduces rows [lo, lo + n_local) of the
 * n_total-entry vector in xslot (greedy when inv_temp <= 0, else Gumbel-max with the unsharded choice's noise per
 * global row), stores its (value, index) key into entry `rank` of the key table in keyslot (a shared slot of
 * 8 x world bytes) here and on every peer, signals `site` once, waits for the other ranks' keys and writes the
 * winner (largest value, lowest index on ties: the unsharded rule) to tokslot. Every rank chooses the same token. */
void tm_cuda_tok_choose_shard(int xslot, unsigned lo, unsigned n_local, unsigned n_total, int tokslot, unsigned max_tokens,
                              float inv_temp, unsigned seed, int stateslot, int keyslot, int site);

/* Device address of a slot (NULL when unreserved); for resident callers and tests. */
void* tm_cuda_tok_slot_ptr(int slot);
/* The lane's stream as a cudaStream_t. */
void* tm_cuda_tok_stream(void);

#ifdef __cplusplus
}
#endif
#endif /* TM_CUDA_SHIM_H */
