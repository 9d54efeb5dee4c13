// include/llama_chain.h — host driver of the GPU decode chain over the token lane.
//
// The decode-lane slice of the reference's model runtime, kept to what the quantized matmul
// path needs (tensormark/llama.h): the slot table (1245-1250), weight registration
// (ensure_gpu_weights 1594-1641), gpu_token_prologue (5716-5770), encode_gpu_token (5774-5930,
// same op order, same fused q|k|v and gate|up segments), forward_gpu_one (5931-5980) and the
// greedy chain API gpu_chain_begin / poll / end / generate_greedy_gpu (6047-6173). Method names,
// argument meaning and error behaviour follow the reference: failures throw std::runtime_error /
// std::invalid_argument, chains need n >= 1 and must fit the context, tokens never leave the GPU
// between the steps of a chain.
//
// Two lanes produce the same tokens:
//   * reference lane: one entry per op through tm_cuda_tok_* exactly as the reference encodes
//     them through tm_metal_tok_* (position passed by value, one host call per op);
//   * graph lane (default for chains): the per-token sequence is encoded ONCE with the chain forms
//     of include/cuda_shim.h (position and token index live in a device "chain state"), captured
//     in a CUDA graph, and replayed per token. RMSNorm and SiLU*up ride in the staging of the
//     following GEMV, the residual adds in the epilogue of the o / down GEMVs, and rope(q),
//     rope(k)->cache, v->cache, attention and the merge of its splits are one launch: 5 launches per layer instead of 14.
//
// Scope: dense Llama-style layers, block-quantized projections (Q8_0/Q4_0/Q4_1/Q5_K/Q6_K),
// GQA attention, greedy choice. Tokenizers, sampling front ends, hybrid/GDN layers, speculative
// decoding and KV paging are outside this path.
#pragma once

#include "cuda_shim.h"
#include "llama_gpu_api.h"
#include "quant.h"

#include <cmath>
#include <cstdlib>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

namespace tmllama {

struct CudaLlamaLayer {
    const void *q = nullptr, *k = nullptr, *v = nullptr, *o = nullptr, *gate = nullptr, *up = nullptr, *down = nullptr;
    const float *rms1 = nullptr, *rms2 = nullptr;              // D floats each (host)
};

struct CudaLlamaDesc {
    int L = 0, D = 0, H = 0, KVH = 0, dh = 0, F = 0, V = 0, ctx = 0;
    float theta = 10000.f, eps = 1e-5f;
    unsigned dt_proj = TM_DT_Q4_0, dt_head = TM_DT_Q6_K, dt_embed = TM_DT_Q4_0;
    const void* embed = nullptr;                               // V x D blocks
    const void* head = nullptr;                                // V x D blocks
    const float* rmsf = nullptr;                               // final norm weights
    const CudaLlamaLayer* layers = nullptr;
    // When every tensor lies inside one host mapping (an mmap'd .tmq), name it here: the mapping is
    // made resident once and all tensors share one weight handle, which is what lets q|k|v and
    // gate|up run as one segmented GEMV each (tensormark/llama.h:5852-5881). Null: one copy per tensor.
    const void* map_base = nullptr;
    size_t map_size = 0;
    // Row sharding over the GPUs of one box, one process per GPU (no counterpart in the reference).
    // With world > 1 this rank holds rows [rank*R/world, (rank+1)*R/world) of gate, up, down and the
    // LM head; every sharded GEMV is followed by tm_cuda_tok_all_gather, so the residual stream, the
    // attention block (q/k/v/o, norms, rope, K/V cache) and the chosen tokens are replicated on every
    // rank. tm_cuda_comm_init must have run. F, D and V must divide by world into multiples of 4 rows.
    int rank = 0, world = 1;
    // How the shards are gathered in the chain forms. true: the GEMVs store their rows into the peers'
    // buffers and the consumers wait on flags (tm_cuda_tok_gemv_xchg; needs tm_cuda_peer_open and one
    // weight mapping, map_base). false: ncclAllGather after each sharded GEMV. The per-op lane
    // (forward_gpu_one, the non-graph chain) always uses ncclAllGather.
    bool peer_gather = false;
};

class CudaLlama {
public:
    enum {
        SLOT_X = 0, SLOT_H = 1, SLOT_QKV = 2, SLOT_AO = 3, SLOT_H2 = 4, SLOT_H2S = 5, SLOT_GU = 6, SLOT_DN = 7,
        SLOT_XF = 8, SLOT_LOGITS = 9, SLOT_PROBS = 10, SLOT_TOK = 11, SLOT_BIAS = 12, SLOT_STATE = 13, SLOT_ACT = 14,
        SLOT_KEYS = 15, SLOT_KC = 100, SLOT_VC = 200
    };

    explicit CudaLlama(const CudaLlamaDesc& d) : d_(d), layers_(d.layers, d.layers + d.L) {
        if (d.L <= 0 || d.D <= 0 || d.H <= 0 || d.KVH <= 0 || d.dh <= 0 || d.F <= 0 || d.V <= 0 || d.ctx <= 0 ||
            d.H % d.KVH || (d.dh & 1) || !d.embed || !d.head || !d.rmsf || !d.layers)
            throw std::invalid_argument("llama: invalid model description");
        if (d.L >= 100) throw std::invalid_argument("llama: the slot table holds at most 99 layers");
        if (d.world < 1 || d.rank < 0 || d.rank >= d.world) throw std::invalid_argument("llama: invalid rank / world");
        if (d.world > 1 && (d.F % (4 * d.world) || d.D % (4 * d.world) || d.V % (4 * d.world)))
            throw std::invalid_argument("llama: F, D and V must split over the ranks into multiples of 4 rows");
        if (!tm_cuda_init(-1)) throw std::runtime_error(std::string("cuda: ") + tm_cuda_last_error());
        logits_.resize((size_t)d.V);
    }
    ~CudaLlama() {
        if (graph_ >= 0) tm_cuda_tok_graph_destroy(graph_);
        if (sgraph_ >= 0) tm_cuda_tok_graph_destroy(sgraph_);
        if (stack_) tm_cuda_llama_destroy(stack_);
    }
    CudaLlama(const CudaLlama&) = delete;
    CudaLlama& operator=(const CudaLlama&) = delete;

    int seen = 0;                                              // tokens in the cache = next position
    const std::vector<float>& logits() const { return logits_; }
    void set_graph_lane(bool on) { use_graph_ = on; }

    // Register every projection once (tensormark/llama.h:1594-1641) and size the packed slots and
    // the K/V caches (5716-5748). Idempotent.
    void gpu_token_prologue() {
        if (ready_) return;
        const int QD = d_.H * d_.dh, KVD = d_.KVH * d_.dh;
        if (d_.world > 1 && d_.peer_gather) {
            if (tm_cuda_peer_world() != d_.world || tm_cuda_peer_rank() != d_.rank)
                throw std::runtime_error("llama: the peer arena does not match the model's rank / world");
            if (!d_.map_base) throw std::invalid_argument("llama: the peer gather needs all tensors in one mapping");
            if (2 * d_.L + 1 > 256) throw std::invalid_argument("llama: too many layers for the exchange sites");
        } else if (d_.world > 1 && (tm_cuda_comm_world() != d_.world || tm_cuda_comm_rank() != d_.rank)) {
            throw std::runtime_error("llama: the communicator does not match the model's rank / world");
        }
        auto reg_rows = [&](const void* p, unsigned dt, int rows, int cols, bool sharded) {
            Handle h{};
            const int mine = sharded ? rows / d_.world : rows;
            const size_t row_bytes = tm_cuda_weight_bytes(dt, 1, (size_t)cols);
            if (!row_bytes) throw std::invalid_argument("llama: tensor shape is not whole blocks");
            const uint8_t* first = (const uint8_t*)p + (sharded ? (size_t)d_.rank * (size_t)mine * row_bytes : 0);
            h.id = tm_cuda_tok_wbuf(first, (size_t)mine * row_bytes, d_.map_base, d_.map_size, d_.map_base ? 1 : 0, &h.woff);
            if (h.id < 0) throw std::runtime_error(std::string("cuda: weight registration failed: ") + tm_cuda_last_error());
            return h;
        };
        auto reg = [&](const void* p, unsigned dt, int rows, int cols) { return reg_rows(p, dt, rows, cols, false); };
        auto reg_shard = [&](const void* p, unsigned dt, int rows, int cols) { return reg_rows(p, dt, rows, cols, d_.world > 1); };
        w_.resize((size_t)d_.L);
        for (int l = 0; l < d_.L; ++l) {
            const CudaLlamaLayer& s = layers_[(size_t)l];
            Registered& r = w_[(size_t)l];
            r.q = reg(s.q, d_.dt_proj, QD, d_.D); r.k = reg(s.k, d_.dt_proj, KVD, d_.D); r.v = reg(s.v, d_.dt_proj, KVD, d_.D);
            r.o = reg(s.o, d_.dt_proj, d_.D, QD);
            r.gate = reg_shard(s.gate, d_.dt_proj, d_.F, d_.D); r.up = reg_shard(s.up, d_.dt_proj, d_.F, d_.D);
            r.down = reg_shard(s.down, d_.dt_proj, d_.D, d_.F);
        }
        embed_ = reg(d_.embed, d_.dt_embed, d_.V, d_.D);
        head_ = reg_shard(d_.head, d_.dt_head, d_.V, d_.D);
        const size_t D4 = (size_t)d_.D * 4;
        // attention scratch: the reference's size, and room for one split per SM of the fused chain kernel
        size_t probs_bytes = (size_t)d_.H * d_.ctx * 4;
        const size_t per_split = (size_t)d_.H * (d_.dh + 2) * 4, want = per_split * (size_t)(tm_cuda_sm_count() / d_.KVH + 1);
        if (probs_bytes < want) probs_bytes = want;
        if (d_.world > 1 && d_.peer_gather &&
            !(tm_cuda_tok_reserve_shared(SLOT_X, D4) && tm_cuda_tok_reserve_shared(SLOT_GU, (size_t)2 * d_.F * 4) &&
              tm_cuda_tok_reserve_shared(SLOT_LOGITS, (size_t)d_.V * 4) && tm_cuda_tok_reserve_shared(SLOT_KEYS, 8 * (size_t)d_.world)))
            throw std::runtime_error(std::string("cuda: shared slot reservation failed: ") + tm_cuda_last_error());
        bool ok = tm_cuda_tok_reserve(SLOT_X, D4) && tm_cuda_tok_reserve(SLOT_H, D4) && tm_cuda_tok_reserve(SLOT_H2, D4) &&
                  tm_cuda_tok_reserve(SLOT_H2S, D4) && tm_cuda_tok_reserve(SLOT_DN, D4) && tm_cuda_tok_reserve(SLOT_XF, D4) &&
                  tm_cuda_tok_reserve(SLOT_QKV, (size_t)(QD + 2 * KVD) * 4) && tm_cuda_tok_reserve(SLOT_AO, (size_t)QD * 4) &&
                  tm_cuda_tok_reserve(SLOT_GU, (size_t)2 * d_.F * 4) && tm_cuda_tok_reserve(SLOT_LOGITS, (size_t)d_.V * 4) &&
                  tm_cuda_tok_reserve(SLOT_PROBS, probs_bytes) && tm_cuda_tok_reserve(SLOT_STATE, 64) &&
                  tm_cuda_tok_reserve(SLOT_ACT, (size_t)d_.F * 4);
        if (!ok) throw std::runtime_error("cuda: packed slot reservation failed");
        const size_t kv = (size_t)d_.KVH * d_.ctx * d_.dh;
        for (int l = 0; l < d_.L; ++l)
            if (!tm_cuda_tok_kv_reserve(SLOT_KC + l, kv) || !tm_cuda_tok_kv_reserve(SLOT_VC + l, kv))
                throw std::runtime_error("cuda: KV cache slot reservation failed");
        ready_ = true;
    }

    // One token's kernels from the first layer norm through lm_head, reference op order
    // (tensormark/llama.h:5818-5924): x in SLOT_X, logits land in SLOT_LOGITS.
    void encode_gpu_token(int pos) {
        const int QD = d_.H * d_.dh, KVD = d_.KVH * d_.dh, REP = d_.H / d_.KVH;
        const float scale = 1.f / std::sqrt((float)d_.dh);
        const unsigned dt = d_.dt_proj;
        for (int l = 0; l < d_.L; ++l) {
            const Registered& r = w_[(size_t)l];
            const CudaLlamaLayer& s = layers_[(size_t)l];
            tm_cuda_tok_rmsnorm(SLOT_X, s.rms1, SLOT_H, (unsigned)d_.D, d_.eps);
            if (same_buffer(r.q, r.k, r.v)) {
                const uint64_t woff[3] = {r.q.woff, r.k.woff, r.v.woff};
                const unsigned rows[3] = {(unsigned)QD, (unsigned)KVD, (unsigned)KVD};
                tm_cuda_tok_gemv_seg_dt(SLOT_H, r.q.id, SLOT_QKV, 0, (unsigned)(QD + 2 * KVD), (unsigned)d_.D, dt, woff, rows, 3);
            } else {
                tm_cuda_tok_gemv_kq(SLOT_H, r.q.id, r.q.woff, SLOT_QKV, 0, (unsigned)QD, (unsigned)d_.D, dt);
                tm_cuda_tok_gemv_kq(SLOT_H, r.k.id, r.k.woff, SLOT_QKV, (size_t)QD * 4, (unsigned)KVD, (unsigned)d_.D, dt);
                tm_cuda_tok_gemv_kq(SLOT_H, r.v.id, r.v.woff, SLOT_QKV, (size_t)(QD + KVD) * 4, (unsigned)KVD, (unsigned)d_.D, dt);
            }
            tm_cuda_tok_rope_q(SLOT_QKV, (unsigned)d_.H, (unsigned)d_.dh, pos, d_.theta);
            tm_cuda_tok_rope_k_cache(SLOT_QKV, (size_t)QD * 4, SLOT_KC + l, (unsigned)d_.KVH, (unsigned)d_.dh, (unsigned)d_.ctx, pos, d_.theta);
            tm_cuda_tok_v_cache(SLOT_QKV, (size_t)(QD + KVD) * 4, SLOT_VC + l, (unsigned)d_.KVH, (unsigned)d_.dh, (unsigned)d_.ctx, pos);
            tm_cuda_tok_attn(SLOT_QKV, SLOT_KC + l, SLOT_VC + l, SLOT_PROBS, SLOT_AO, (unsigned)QD, (unsigned)d_.H, (unsigned)d_.KVH,
                             (unsigned)d_.dh, (unsigned)d_.ctx, pos + 1, scale, (unsigned)REP);
            tm_cuda_tok_gemv_kq(SLOT_AO, r.o.id, r.o.woff, SLOT_H2, 0, (unsigned)d_.D, (unsigned)QD, dt);
            tm_cuda_tok_add(SLOT_X, SLOT_H2, (unsigned)d_.D);
            tm_cuda_tok_rmsnorm(SLOT_X, s.rms2, SLOT_H2S, (unsigned)d_.D, d_.eps);
            if (d_.world > 1) {
                const unsigned Fs = (unsigned)(d_.F / d_.world), Ds = (unsigned)(d_.D / d_.world);
                tm_cuda_tok_gemv_kq(SLOT_H2S, r.gate.id, r.gate.woff, SLOT_GU, 0, Fs, (unsigned)d_.D, dt);
                tm_cuda_tok_gemv_kq(SLOT_H2S, r.up.id, r.up.woff, SLOT_GU, (size_t)Fs * 4, Fs, (unsigned)d_.D, dt);
                tm_cuda_tok_silu_mul(SLOT_GU, 0, SLOT_GU, (size_t)Fs * 4, Fs);
                tm_cuda_tok_all_gather(SLOT_GU, 0, SLOT_ACT, 0, Fs);
                tm_cuda_tok_gemv_kq(SLOT_ACT, r.down.id, r.down.woff, SLOT_DN, (size_t)d_.rank * Ds * 4, Ds, (unsigned)d_.F, dt);
                tm_cuda_tok_all_gather(SLOT_DN, (size_t)d_.rank * Ds * 4, SLOT_DN, 0, Ds);
                tm_cuda_tok_add(SLOT_X, SLOT_DN, (unsigned)d_.D);
                continue;
            }
            tm_cuda_tok_gemv_kq(SLOT_H2S, r.gate.id, r.gate.woff, SLOT_GU, 0, (unsigned)d_.F, (unsigned)d_.D, dt);
            tm_cuda_tok_gemv_kq(SLOT_H2S, r.up.id, r.up.woff, SLOT_GU, (size_t)d_.F * 4, (unsigned)d_.F, (unsigned)d_.D, dt);
            tm_cuda_tok_silu_mul(SLOT_GU, 0, SLOT_GU, (size_t)d_.F * 4, (unsigned)d_.F);
            tm_cuda_tok_gemv_kq(SLOT_GU, r.down.id, r.down.woff, SLOT_DN, 0, (unsigned)d_.D, (unsigned)d_.F, dt);
            tm_cuda_tok_add(SLOT_X, SLOT_DN, (unsigned)d_.D);
        }
        tm_cuda_tok_rmsnorm(SLOT_X, d_.rmsf, SLOT_XF, (unsigned)d_.D, d_.eps);
        if (d_.world > 1) {
            const unsigned Vs = (unsigned)(d_.V / d_.world);
            tm_cuda_tok_gemv_kq(SLOT_XF, head_.id, head_.woff, SLOT_LOGITS, (size_t)d_.rank * Vs * 4, Vs, (unsigned)d_.D, d_.dt_head);
            tm_cuda_tok_all_gather(SLOT_LOGITS, (size_t)d_.rank * Vs * 4, SLOT_LOGITS, 0, Vs);
            return;
        }
        tm_cuda_tok_gemv_kq(SLOT_XF, head_.id, head_.woff, SLOT_LOGITS, 0, (unsigned)d_.V, (unsigned)d_.D, d_.dt_head);
    }

    // Chain form of the same token: position and token index come from SLOT_STATE on the device,
    // norms / SiLU / residuals are folded into the GEMVs. Encoded once and captured.
    void encode_chain_token(unsigned max_tokens) {
        const int QD = d_.H * d_.dh, KVD = d_.KVH * d_.dh;
        const float scale = 1.f / std::sqrt((float)d_.dh);
        const unsigned dt = d_.dt_proj;
        tm_cuda_tok_embed_at(SLOT_TOK, embed_.id, embed_.woff, SLOT_X, (unsigned)d_.D, d_.dt_embed, max_tokens, SLOT_STATE);
        if (d_.world > 1 && d_.peer_gather) { encode_chain_token_peer(max_tokens); return; }
        for (int l = 0; l < d_.L; ++l) {
            const Registered& r = w_[(size_t)l];
            const CudaLlamaLayer& s = layers_[(size_t)l];
            const unsigned qkv_rows[3] = {(unsigned)QD, (unsigned)KVD, (unsigned)KVD};
            if (same_buffer(r.q, r.k, r.v)) {
                const uint64_t woff[3] = {r.q.woff, r.k.woff, r.v.woff};
                tm_cuda_tok_gemv_fused(SLOT_X, 0, 1, 0, 0, s.rms1, d_.eps, r.q.id, SLOT_QKV, 0, (unsigned)(QD + 2 * KVD), (unsigned)d_.D, dt, woff, qkv_rows, 3, 0);
            } else {
                const Handle* hs[3] = {&r.q, &r.k, &r.v};
                size_t yoff = 0;
                for (int i = 0; i < 3; ++i) {
                    tm_cuda_tok_gemv_fused(SLOT_X, 0, 1, 0, 0, s.rms1, d_.eps, hs[i]->id, SLOT_QKV, yoff, qkv_rows[i], (unsigned)d_.D, dt, &hs[i]->woff, &qkv_rows[i], 1, 0);
                    yoff += (size_t)qkv_rows[i] * 4;
                }
            }
            tm_cuda_tok_attn_fused_at(SLOT_QKV, SLOT_KC + l, SLOT_VC + l, SLOT_PROBS, SLOT_AO, (unsigned)d_.H, (unsigned)d_.KVH,
                                      (unsigned)d_.dh, (unsigned)d_.ctx, scale, d_.theta, SLOT_STATE);
            const unsigned Dn = (unsigned)d_.D, Fn = (unsigned)d_.F;
            tm_cuda_tok_gemv_fused(SLOT_AO, 0, 0, 0, 0, nullptr, 0.f, r.o.id, SLOT_X, 0, Dn, (unsigned)QD, dt, &r.o.woff, &Dn, 1, 1);
            if (d_.world > 1) {
                // this rank's rows of gate|up -> SiLU*up on the shard -> gather the activation; this rank's
                // rows of down accumulate into its slice of the residual, which is then gathered in place
                const unsigned Fs = Fn / (unsigned)d_.world, Ds = Dn / (unsigned)d_.world;
                if (same_buffer(r.gate, r.up, r.up)) {
                    const uint64_t woff[2] = {r.gate.woff, r.up.woff};
                    const unsigned rows[2] = {Fs, Fs};
                    tm_cuda_tok_gemv_fused(SLOT_X, 0, 1, 0, 0, s.rms2, d_.eps, r.gate.id, SLOT_GU, 0, 2 * Fs, Dn, dt, woff, rows, 2, 0);
                } else {
                    tm_cuda_tok_gemv_fused(SLOT_X, 0, 1, 0, 0, s.rms2, d_.eps, r.gate.id, SLOT_GU, 0, Fs, Dn, dt, &r.gate.woff, &Fs, 1, 0);
                    tm_cuda_tok_gemv_fused(SLOT_X, 0, 1, 0, 0, s.rms2, d_.eps, r.up.id, SLOT_GU, (size_t)Fs * 4, Fs, Dn, dt, &r.up.woff, &Fs, 1, 0);
                }
                tm_cuda_tok_silu_mul(SLOT_GU, 0, SLOT_GU, (size_t)Fs * 4, Fs);
                tm_cuda_tok_all_gather(SLOT_GU, 0, SLOT_ACT, 0, Fs);
                tm_cuda_tok_gemv_fused(SLOT_ACT, 0, 0, 0, 0, nullptr, 0.f, r.down.id, SLOT_X, (size_t)d_.rank * Ds * 4, Ds, Fn, dt, &r.down.woff, &Ds, 1, 1);
                tm_cuda_tok_all_gather(SLOT_X, (size_t)d_.rank * Ds * 4, SLOT_X, 0, Ds);
                continue;
            }
            if (same_buffer(r.gate, r.up, r.up)) {
                const uint64_t woff[2] = {r.gate.woff, r.up.woff};
                const unsigned rows[2] = {Fn, Fn};
                tm_cuda_tok_gemv_fused(SLOT_X, 0, 1, 0, 0, s.rms2, d_.eps, r.gate.id, SLOT_GU, 0, 2 * Fn, Dn, dt, woff, rows, 2, 0);
            } else {
                tm_cuda_tok_gemv_fused(SLOT_X, 0, 1, 0, 0, s.rms2, d_.eps, r.gate.id, SLOT_GU, 0, Fn, Dn, dt, &r.gate.woff, &Fn, 1, 0);
                tm_cuda_tok_gemv_fused(SLOT_X, 0, 1, 0, 0, s.rms2, d_.eps, r.up.id, SLOT_GU, (size_t)Fn * 4, Fn, Dn, dt, &r.up.woff, &Fn, 1, 0);
            }
            tm_cuda_tok_gemv_fused(SLOT_GU, 0, 2, SLOT_GU, (size_t)Fn * 4, nullptr, 0.f, r.down.id, SLOT_X, 0, Dn, Fn, dt, &r.down.woff, &Dn, 1, 1);
        }
        const unsigned Vn = (unsigned)d_.V;
        if (d_.world > 1) {
            const unsigned Vs = Vn / (unsigned)d_.world;
            tm_cuda_tok_gemv_fused(SLOT_X, 0, 1, 0, 0, d_.rmsf, d_.eps, head_.id, SLOT_LOGITS, (size_t)d_.rank * Vs * 4, Vs, (unsigned)d_.D, d_.dt_head, &head_.woff, &Vs, 1, 0);
            tm_cuda_tok_all_gather(SLOT_LOGITS, (size_t)d_.rank * Vs * 4, SLOT_LOGITS, 0, Vs);
        } else {
            tm_cuda_tok_gemv_fused(SLOT_X, 0, 1, 0, 0, d_.rmsf, d_.eps, head_.id, SLOT_LOGITS, 0, Vn, (unsigned)d_.D, d_.dt_head, &head_.woff, &Vn, 1, 0);
        }
        if (inv_temp_ > 0.f) tm_cuda_tok_sample_at(SLOT_LOGITS, SLOT_TOK, Vn, max_tokens, inv_temp_, seed_, SLOT_STATE, -1);
        else tm_cuda_tok_argmax_at(SLOT_LOGITS, SLOT_TOK, Vn, max_tokens, SLOT_STATE);
        tm_cuda_tok_advance(SLOT_STATE);
    }

    // The chain token of a row-sharded model with the gather fused into the GEMVs. Sites: 2l = the
    // activation of layer l, 2l+1 = the residual after layer l, 2L = the logits. A GEMV that computes
    // a shard writes its rows at their place in the full vector, here and on every peer; the first
    // kernel that reads a gathered vector waits for the other ranks' rows.
    void encode_chain_token_peer(unsigned max_tokens) {
        const int QD = d_.H * d_.dh, KVD = d_.KVH * d_.dh;
        const float scale = 1.f / std::sqrt((float)d_.dh);
        const unsigned dt = d_.dt_proj, Dn = (unsigned)d_.D, Fn = (unsigned)d_.F, Vn = (unsigned)d_.V;
        const unsigned Fs = Fn / (unsigned)d_.world, Ds = Dn / (unsigned)d_.world, Vs = Vn / (unsigned)d_.world;
        const size_t rk = (size_t)d_.rank;
        for (int l = 0; l < d_.L; ++l) {
            const Registered& r = w_[(size_t)l];
            const CudaLlamaLayer& s = layers_[(size_t)l];
            const unsigned qkv_rows[3] = {(unsigned)QD, (unsigned)KVD, (unsigned)KVD};
            const uint64_t qkv_woff[3] = {r.q.woff, r.k.woff, r.v.woff};
            const size_t qkv_yoff[3] = {0, (size_t)QD * 4, (size_t)(QD + KVD) * 4};
            tm_cuda_tok_gemv_xchg(SLOT_X, 0, 1, 0, 0, s.rms1, d_.eps, r.q.id, SLOT_QKV, qkv_yoff, (unsigned)(QD + 2 * KVD), Dn, dt,
                                  qkv_woff, qkv_rows, 3, 0, l > 0 ? 2 * l - 1 : -1, -1, SLOT_STATE);
            tm_cuda_tok_attn_fused_at(SLOT_QKV, SLOT_KC + l, SLOT_VC + l, SLOT_PROBS, SLOT_AO, (unsigned)d_.H, (unsigned)d_.KVH,
                                      (unsigned)d_.dh, (unsigned)d_.ctx, scale, d_.theta, SLOT_STATE);
            tm_cuda_tok_gemv_fused(SLOT_AO, 0, 0, 0, 0, nullptr, 0.f, r.o.id, SLOT_X, 0, Dn, (unsigned)QD, dt, &r.o.woff, &Dn, 1, 1);
            const uint64_t gu_woff[2] = {r.gate.woff, r.up.woff};
            const unsigned gu_rows[2] = {Fs, Fs};
            const size_t gu_yoff[2] = {rk * Fs * 4, ((size_t)Fn + rk * Fs) * 4};
            tm_cuda_tok_gemv_xchg(SLOT_X, 0, 1, 0, 0, s.rms2, d_.eps, r.gate.id, SLOT_GU, gu_yoff, 2 * Fs, Dn, dt, gu_woff, gu_rows, 2, 0,
                                  -1, 2 * l, SLOT_STATE);
            const size_t dn_yoff[1] = {rk * Ds * 4};
            tm_cuda_tok_gemv_xchg(SLOT_GU, 0, 2, SLOT_GU, (size_t)Fn * 4, nullptr, 0.f, r.down.id, SLOT_X, dn_yoff, Ds, Fn, dt, &r.down.woff, &Ds, 1, 1,
                                  2 * l, 2 * l + 1, SLOT_STATE);
        }
        const size_t hd_yoff[1] = {rk * Vs * 4};
        if (gather_logits_) {
            tm_cuda_tok_gemv_xchg(SLOT_X, 0, 1, 0, 0, d_.rmsf, d_.eps, head_.id, SLOT_LOGITS, hd_yoff, Vs, Dn, d_.dt_head, &head_.woff, &Vs, 1, 0,
                                  2 * d_.L - 1, 2 * d_.L, SLOT_STATE);
            if (inv_temp_ > 0.f) tm_cuda_tok_sample_at(SLOT_LOGITS, SLOT_TOK, Vn, max_tokens, inv_temp_, seed_, SLOT_STATE, 2 * d_.L);
            else tm_cuda_tok_argmax_xchg(SLOT_LOGITS, SLOT_TOK, Vn, max_tokens, SLOT_STATE, 2 * d_.L);
        } else {
            // The logits stay where they are computed: every rank chooses over its own rows and only the g (value, index)
            // keys are exchanged (tie rule of the unsharded choice, tensormark/metal.h:2335: the lowest index wins).
            tm_cuda_tok_gemv_xchg(SLOT_X, 0, 1, 0, 0, d_.rmsf, d_.eps, head_.id, SLOT_LOGITS, hd_yoff, Vs, Dn, d_.dt_head, &head_.woff, &Vs, 1, 0,
                                  2 * d_.L - 1, -1, SLOT_STATE);
            tm_cuda_tok_choose_shard(SLOT_LOGITS, (unsigned)(rk * Vs), Vs, Vn, SLOT_TOK, max_tokens, inv_temp_ > 0.f ? inv_temp_ : 0.f, seed_, SLOT_STATE,
                                     SLOT_KEYS, 2 * d_.L);
        }
        tm_cuda_tok_advance(SLOT_STATE);
    }

    // Rows of the logits vector that the graph chain leaves valid on this rank: all of them, except for a row-sharded
    // model whose ranks exchange only their choices (then this rank's rows of the head).
    void chain_logit_rows(int& lo, int& hi) const {
        lo = 0; hi = d_.V;
        if (d_.world > 1 && d_.peer_gather && !gather_logits_) { lo = d_.rank * (d_.V / d_.world); hi = lo + d_.V / d_.world; }
    }

    // One forward at position `seen`: logits of that token (tensormark/llama.h:5931-5980).
    std::vector<float>& forward_gpu_one(int tok) {
        if (tok < 0 || tok >= d_.V) throw std::invalid_argument("llama: token id out of range");
        if (seen >= d_.ctx) throw std::invalid_argument("llama: context is full");
        gpu_token_prologue();
        if (seen < stack_rows_) stack_rows_ = seen;     // the decode lane writes K/V rows from here on: the layer stack's own rows beyond are stale
        const unsigned t = (unsigned)tok;
        if (!tm_cuda_tok_upload(SLOT_TOK, 0, &t, sizeof t)) throw std::runtime_error("cuda: token upload failed");
        if (!tm_cuda_tok_begin()) throw std::runtime_error("cuda: token begin failed");
        tm_cuda_tok_embed_kq(SLOT_TOK, 0, embed_.id, embed_.woff, SLOT_X, (unsigned)d_.D, d_.dt_embed);
        encode_gpu_token(seen);
        if (!tm_cuda_tok_end(SLOT_LOGITS, logits_.data(), (unsigned)d_.V))
            throw std::runtime_error(std::string("cuda: token execution failed: ") + tm_cuda_last_error());
        seen += 1;
        return logits_;
    }

    // Greedy chain (tensormark/llama.h:6047-6165): feeds `first` at the current position and
    // chooses n tokens on the GPU, chosen tokens 0..n-2 being fed by the following steps.
    // The same chain with Gumbel-max sampling on the GPU (tensormark/metal.h:2349-2379: noise = hash of seed, token
    // index and vocabulary index; inv_temp = 1 / temperature). Every rank of a sharded model draws the same tokens.
    void gpu_chain_begin_sampled(int first, int n, float inv_temp, unsigned seed) {
        if (!(inv_temp > 0.f) || !std::isfinite(inv_temp)) throw std::invalid_argument("llama: sampling needs a positive, finite inverse temperature");
        inv_temp_ = inv_temp; seed_ = seed;
        try { gpu_chain_begin(first, n); } catch (...) { inv_temp_ = 0.f; throw; }
        inv_temp_ = 0.f;                                       // the launches are enqueued; later chains are greedy again
    }
    void gpu_chain_begin(int first, int n) {
        if (n <= 0) throw std::invalid_argument("llama: chain needs n >= 1");
        if (first < 0 || first >= d_.V) throw std::invalid_argument("llama: token id out of range");
        if (seen + n > d_.ctx) throw std::invalid_argument("llama: chain exceeds context");
        if (chain_n_) throw std::runtime_error("llama: chain already running");
        gpu_token_prologue();
        if (seen < stack_rows_) stack_rows_ = seen;     // the decode lane writes K/V rows from here on: the layer stack's own rows beyond are stale
        const unsigned cap = (unsigned)d_.ctx + 1;
        std::vector<unsigned> toks((size_t)cap, 0xFFFFFFFFu);
        toks[0] = (unsigned)first;
        if (!tm_cuda_tok_reserve(SLOT_TOK, sizeof(unsigned) * (size_t)cap) ||
            !tm_cuda_tok_upload(SLOT_TOK, 0, toks.data(), sizeof(unsigned) * (size_t)cap))
            throw std::runtime_error("cuda: token slot upload failed");
        if (use_graph_) {
            run_graph(n, /*forced=*/1);
        } else {
            for (int i = 0; i < n; ++i) {
                if (!tm_cuda_tok_begin()) throw std::runtime_error("cuda: token begin failed");
                tm_cuda_tok_embed_kq(SLOT_TOK, (unsigned)i, embed_.id, embed_.woff, SLOT_X, (unsigned)d_.D, d_.dt_embed);
                encode_gpu_token(seen + i);
                if (inv_temp_ > 0.f) tm_cuda_tok_sample(SLOT_LOGITS, SLOT_TOK, (unsigned)(i + 1), (unsigned)d_.V, inv_temp_, seed_);
                else tm_cuda_tok_argmax(SLOT_LOGITS, SLOT_TOK, (unsigned)(i + 1), (unsigned)d_.V);
                if (!tm_cuda_tok_end_async()) throw std::runtime_error("cuda: token commit failed");
            }
        }
        chain_n_ = n; chain_seen0_ = seen;
    }
    // Feed n known tokens (a prompt) through the graph lane, one position each; returns the token the
    // model chooses after the last one. The reference prefills with its batched layer stack
    // (tensormark/llama.h:6305-6352); on this path a prompt is decoded token by token, which leaves the
    // K/V caches in exactly the state the chain continues from.
    int gpu_feed(const int* toks, int n) {
        if (n <= 0) throw std::invalid_argument("llama: feed needs n >= 1");
        if (seen + n > d_.ctx) throw std::invalid_argument("llama: prompt exceeds context");
        if (chain_n_) throw std::runtime_error("llama: chain already running");
        gpu_token_prologue();
        if (seen < stack_rows_) stack_rows_ = seen;     // the decode lane writes K/V rows from here on: the layer stack's own rows beyond are stale
        const unsigned cap = (unsigned)d_.ctx + 1;
        std::vector<unsigned> t((size_t)cap, 0xFFFFFFFFu);
        for (int i = 0; i < n; ++i) {
            if (toks[i] < 0 || toks[i] >= d_.V) throw std::invalid_argument("llama: token id out of range");
            t[(size_t)i] = (unsigned)toks[i];
        }
        if (!tm_cuda_tok_reserve(SLOT_TOK, sizeof(unsigned) * (size_t)cap) ||
            !tm_cuda_tok_upload(SLOT_TOK, 0, t.data(), sizeof(unsigned) * (size_t)cap))
            throw std::runtime_error("cuda: token slot upload failed");
        run_graph(n, /*forced=*/n);
        unsigned next = 0;
        if (!tm_cuda_tok_wait_pending() || !tm_cuda_tok_download(SLOT_TOK, sizeof(unsigned) * (size_t)n, &next, sizeof next))
            throw std::runtime_error(std::string("cuda: prompt execution failed: ") + tm_cuda_last_error());
        seen += n;
        return (int)next;
    }

    // A prompt of n >= 3 tokens: the first n - 1 through the batched layer stack (tensormark/llama.h:6305-6352: embed
    // the rows on the host, tm_*_llama_prefill), the stack's K/V rows into the decode lane's caches on the device, and
    // the last token through the decode lane, which leaves its logits and the model's next token exactly as gpu_feed
    // does. Returns that token. With a row-sharded model every rank runs the stack on the whole prompt (attention and
    // its K/V caches are replicated); only the last token's FFN and LM head are sharded.
    int gpu_prefill(const int* toks, int n) {
        if (n < 3) throw std::invalid_argument("llama: the layer stack takes prompts of three or more tokens");
        if (seen + n > d_.ctx) throw std::invalid_argument("llama: prompt exceeds context");
        if (chain_n_) throw std::runtime_error("llama: chain already running");
        gpu_token_prologue();
        ensure_stack();
        // The stack's caches hold the rows the stack itself computed ([0, stack_rows_)). After tokens that went through the
        // decode lane its rows are behind: such a prompt continues token by token.
        if (seen > stack_rows_) return gpu_feed(toks, n);
        const int m = n - 1;
        for (int i = 0; i < n; ++i)
            if (toks[i] < 0 || toks[i] >= d_.V) throw std::invalid_argument("llama: token id out of range");
        // The embedding rows are gathered on the device from the table the decode lane has registered, and the residual
        // stream after the last layer is of no use here (the prompt's last token goes through the decode lane), so
        // nothing but the token ids crosses the bus.
        if (!tm_cuda_llama_prefill_begin_tokens(stack_, toks, m, seen, embed_.id, embed_.woff, d_.V, d_.dt_embed) || !tm_cuda_llama_prefill_end())
            throw std::runtime_error(std::string("cuda: layer stack prefill failed: ") + tm_cuda_last_error());
        for (int l = 0; l < d_.L; ++l)
            if (!tm_cuda_llama_kv_to_slots(stack_, l, SLOT_KC + l, SLOT_VC + l, seen, m))
                throw std::runtime_error(std::string("cuda: K/V hand-over failed: ") + tm_cuda_last_error());
        seen += m;
        stack_rows_ = seen;
        return gpu_feed(toks + m, 1);
    }
    double last_prefill_gpu_ms() const { return tm_cuda_llama_prefill_gpu_ms(); }
    // Creates the layer stack ahead of the first gpu_prefill (it is otherwise created by it).
    void gpu_prefill_prepare(int max_tokens = 0) {
        gpu_token_prologue();
        ensure_stack();
        if (max_tokens >= 3 && !tm_cuda_llama_reserve(stack_, max_tokens - 1))
            throw std::runtime_error(std::string("cuda: layer stack buffers: ") + tm_cuda_last_error());
    }

    // Chosen token i as soon as it has landed, -1 while pending.
    int gpu_chain_poll(int i) const {
        if (i < 0 || i >= chain_n_) return -1;
        const unsigned t = tm_cuda_tok_peek(SLOT_TOK, (unsigned)(i + 1));
        return t == 0xFFFFFFFFu ? -1 : (int)t;
    }
    // The n chosen tokens (the last one not yet fed). keep >= 0: the caller stopped at chosen
    // token `keep`; the cache position becomes seen0 + keep + 1.
    std::vector<int> gpu_chain_end(int keep = -1) {
        std::vector<int> out;
        if (!chain_n_) return out;
        if (!tm_cuda_tok_wait_pending()) throw std::runtime_error(std::string("cuda: chained token execution failed: ") + tm_cuda_last_error());
        std::vector<unsigned> toks((size_t)chain_n_);
        if (!tm_cuda_tok_download(SLOT_TOK, sizeof(unsigned), toks.data(), sizeof(unsigned) * (size_t)chain_n_) ||
            !tm_cuda_tok_download(SLOT_LOGITS, 0, logits_.data(), sizeof(float) * (size_t)d_.V))
            throw std::runtime_error("cuda: chained result download failed");
        out.assign(toks.begin(), toks.end());
        seen = keep < 0 ? chain_seen0_ + chain_n_ : chain_seen0_ + keep + 1;
        chain_n_ = 0;
        return out;
    }
    // n forwards (first + n-1 chosen tokens); returns the n-1 chosen tokens that were fed.
    std::vector<int> generate_greedy_gpu(int first, int n) {
        gpu_chain_begin(first, n);
        std::vector<int> t = gpu_chain_end();
        t.pop_back();
        return t;
    }

private:
    // The layer stack of this model. Its K/V rows stay on the device (null kc / vc: tm_cuda_llama_kv_to_slots hands them to
    // the decode lane), which spares a prompt the copy of every row to host arrays nobody reads.
    void ensure_stack() {
        if (stack_) return;
        stack_layers_.resize((size_t)d_.L);
        for (int l = 0; l < d_.L; ++l) {
            const CudaLlamaLayer& s = layers_[(size_t)l];
            tm_llama_gpu_layer& g = stack_layers_[(size_t)l];
            g = tm_llama_gpu_layer{};
            g.q = s.q; g.k = s.k; g.v = s.v; g.o = s.o; g.gate = s.gate; g.up = s.up; g.down = s.down;
            g.rms1 = s.rms1; g.rms2 = s.rms2;
        }
        tm_llama_gpu_desc gd{};
        gd.L = d_.L; gd.D = d_.D; gd.H = d_.H; gd.KVH = d_.KVH; gd.dh = d_.dh; gd.F = d_.F; gd.ctx = d_.ctx;
        gd.theta = d_.theta; gd.eps = d_.eps; gd.map_base = d_.map_base; gd.map_size = d_.map_size; gd.layers = stack_layers_.data();
        stack_ = tm_cuda_llama_create_dt(&gd, d_.dt_proj);
        if (!stack_) throw std::runtime_error(std::string("cuda: layer stack creation failed: ") + tm_cuda_last_error());
    }

    // Launch the captured token graph `n` times from position `seen`; the first `forced` entries of the
    // token slot are inputs. The very first call runs one token eagerly (which creates every cached
    // resource) and captures the second encoding.
    void run_graph(int n, int forced) {
        const unsigned cap = (unsigned)d_.ctx + 1;
        const int st[3] = {seen, 0, forced};
        if (!tm_cuda_tok_upload(SLOT_STATE, 0, st, sizeof st)) throw std::runtime_error("cuda: chain state upload failed");
        int left = n;
        // one graph for greedy chains, one for sampled chains (it holds the temperature and the seed)
        const bool sampling = inv_temp_ > 0.f;
        int& g = sampling ? sgraph_ : graph_;
        if (sampling && g >= 0 && (sg_inv_temp_ != inv_temp_ || sg_seed_ != seed_)) { tm_cuda_tok_graph_destroy(g); g = -1; }
        if (g < 0) {
            if (!tm_cuda_tok_begin()) throw std::runtime_error("cuda: token begin failed");
            encode_chain_token(cap);
            if (!tm_cuda_tok_flush()) throw std::runtime_error(std::string("cuda: chain token failed: ") + tm_cuda_last_error());
            if (!tm_cuda_tok_graph_begin()) throw std::runtime_error("cuda: graph capture failed");
            encode_chain_token(cap);
            g = tm_cuda_tok_graph_end();
            if (g < 0) throw std::runtime_error(std::string("cuda: graph capture failed: ") + tm_cuda_last_error());
            if (sampling) { sg_inv_temp_ = inv_temp_; sg_seed_ = seed_; }
            left -= 1;
        }
        if (left > 0 && !tm_cuda_tok_graph_launch(g, (unsigned)left)) throw std::runtime_error("cuda: graph launch failed");
    }

    struct Handle { int id = -1; uint64_t woff = 0; };
    struct Registered { Handle q, k, v, o, gate, up, down; };
    static bool same_buffer(const Handle& a, const Handle& b, const Handle& c) { return a.id == b.id && b.id == c.id; }

    CudaLlamaDesc d_;
    std::vector<CudaLlamaLayer> layers_;
    std::vector<Registered> w_;
    Handle embed_, head_;
    std::vector<float> logits_;
    bool ready_ = false, use_graph_ = true;
    int graph_ = -1, sgraph_ = -1, chain_n_ = 0, chain_seen0_ = 0;
    void* stack_ = nullptr;
    std::vector<tm_llama_gpu_layer> stack_layers_;
    int stack_rows_ = 0;                                       // positions [0, stack_rows_) of the stack's K/V caches match this sequence
    float inv_temp_ = 0.f, sg_inv_temp_ = 0.f;                 // > 0 only while a sampled chain is being encoded
    // Peer-gather chain: true = the LM head's rows are gathered on every rank before the choice (every rank then holds
    // all logits of the last step), false = only the ranks' (value, index) keys travel. TM_CUDA_GATHER_LOGITS=1 selects
    // the former for callers that read the chain's logits.
    bool gather_logits_ = [] { const char* e = std::getenv("TM_CUDA_GATHER_LOGITS"); return e && *e == '1'; }();
    unsigned seed_ = 0, sg_seed_ = 0;
};

}  // namespace tmllama
