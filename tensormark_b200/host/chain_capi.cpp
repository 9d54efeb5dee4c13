// chain_capi.cpp — C entry points over tmllama::CudaLlama (include/llama_chain.h).
//
// The decode-chain driver is a C++ class, as its counterpart in the reference is; this file
// gives it a flat C surface so that programs without a C++ toolchain at hand (the Python tests
// and the benchmark, through ctypes) can drive the same object. No arithmetic lives here.
#include "llama_chain.h"
#include "tmq_reader.h"

#include <cstring>
#include <memory>
#include <string>

namespace {
thread_local std::string g_err;
struct Holder {
    std::vector<tmllama::CudaLlamaLayer> layers;
    std::unique_ptr<tmllama::CudaLlama> m;
};
}  // namespace

#define TMCHAIN_API extern "C" __attribute__((visibility("default")))

TMCHAIN_API const char* tmchain_error(void) { return g_err.c_str(); }

// cfg = {L, D, H, KVH, dh, F, V, ctx, dt_proj, dt_head, dt_embed, rank, world, peer_gather}; layer_ptrs holds, per layer,
// q, k, v, o, gate, up, down, rms1, rms2 (9 pointers).
TMCHAIN_API void* tmchain_create(const int* cfg, float theta, float eps, const void* embed, const void* head,
                                 const float* rmsf, const void* const* layer_ptrs, const void* map_base, size_t map_size) {
    try {
        auto h = std::make_unique<Holder>();
        tmllama::CudaLlamaDesc d;
        d.L = cfg[0]; d.D = cfg[1]; d.H = cfg[2]; d.KVH = cfg[3]; d.dh = cfg[4]; d.F = cfg[5]; d.V = cfg[6]; d.ctx = cfg[7];
        d.dt_proj = (unsigned)cfg[8]; d.dt_head = (unsigned)cfg[9]; d.dt_embed = (unsigned)cfg[10];
        d.theta = theta; d.eps = eps; d.embed = embed; d.head = head; d.rmsf = rmsf;
        d.map_base = map_base; d.map_size = map_size;
        d.rank = cfg[11]; d.world = cfg[12]; d.peer_gather = cfg[13] != 0;
        h->layers.resize((size_t)(d.L > 0 ? d.L : 0));
        for (int l = 0; l < d.L; ++l) {
            const void* const* p = layer_ptrs + 9 * l;
            tmllama::CudaLlamaLayer& s = h->layers[(size_t)l];
            s.q = p[0]; s.k = p[1]; s.v = p[2]; s.o = p[3]; s.gate = p[4]; s.up = p[5]; s.down = p[6];
            s.rms1 = (const float*)p[7]; s.rms2 = (const float*)p[8];
        }
        d.layers = h->layers.data();
        h->m = std::make_unique<tmllama::CudaLlama>(d);
        return h.release();
    } catch (const std::exception& e) { g_err = e.what(); return nullptr; }
}
// Also drops the lane's weight registrations: they are keyed by the host addresses of this model's tensors.
TMCHAIN_API void tmchain_destroy(void* p) {
    delete static_cast<Holder*>(p);                        // the layer stack goes first: it points into the resident weights
    tm_cuda_release_weights();
}
TMCHAIN_API int tmchain_seen(void* p) { return static_cast<Holder*>(p)->m->seen; }
TMCHAIN_API void tmchain_set_seen(void* p, int seen) { static_cast<Holder*>(p)->m->seen = seen; }

TMCHAIN_API int tmchain_forward(void* p, int tok, float* logits) {
    try {
        auto& m = *static_cast<Holder*>(p)->m;
        const std::vector<float>& l = m.forward_gpu_one(tok);
        if (logits) std::memcpy(logits, l.data(), l.size() * sizeof(float));
        return 1;
    } catch (const std::exception& e) { g_err = e.what(); return 0; }
}
// n forwards starting with `first`; out receives the n chosen tokens, last_logits the logits of the last step.
TMCHAIN_API int tmchain_greedy(void* p, int first, int n, int* out, float* last_logits, int use_graph) {
    try {
        auto& m = *static_cast<Holder*>(p)->m;
        m.set_graph_lane(use_graph != 0);
        m.gpu_chain_begin(first, n);
        const std::vector<int> t = m.gpu_chain_end();
        for (size_t i = 0; i < t.size(); ++i) out[i] = t[i];
        if (last_logits) std::memcpy(last_logits, m.logits().data(), m.logits().size() * sizeof(float));
        return 1;
    } catch (const std::exception& e) { g_err = e.what(); return 0; }
}
// Begin a chain without waiting (for timing and for polling); end it with tmchain_chain_end.
TMCHAIN_API int tmchain_chain_begin(void* p, int first, int n, int use_graph) {
    try {
        auto& m = *static_cast<Holder*>(p)->m;
        m.set_graph_lane(use_graph != 0);
        m.gpu_chain_begin(first, n);
        return 1;
    } catch (const std::exception& e) { g_err = e.what(); return 0; }
}
// The same with Gumbel-max sampling (inv_temp = 1 / temperature).
TMCHAIN_API int tmchain_chain_begin_sampled(void* p, int first, int n, float inv_temp, unsigned seed, int use_graph) {
    try {
        auto& m = *static_cast<Holder*>(p)->m;
        m.set_graph_lane(use_graph != 0);
        m.gpu_chain_begin_sampled(first, n, inv_temp, seed);
        return 1;
    } catch (const std::exception& e) { g_err = e.what(); return 0; }
}
TMCHAIN_API int tmchain_chain_poll(void* p, int i) { return static_cast<Holder*>(p)->m->gpu_chain_poll(i); }
TMCHAIN_API int tmchain_chain_end(void* p, int keep, int* out, int cap) {
    try {
        const std::vector<int> t = static_cast<Holder*>(p)->m->gpu_chain_end(keep);
        for (size_t i = 0; i < t.size() && (int)i < cap; ++i) out[i] = t[i];
        return (int)t.size();
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}
// The logits of the most recent forward / finished chain (V floats).
TMCHAIN_API int tmchain_logits(void* p, float* out) {
    const std::vector<float>& l = static_cast<Holder*>(p)->m->logits();
    std::memcpy(out, l.data(), l.size() * sizeof(float));
    return (int)l.size();
}
// Rows [lo, hi) of that vector that a finished graph chain left valid on this rank (all, unless the ranks of a
// row-sharded model exchanged only their choices).
TMCHAIN_API void tmchain_logit_rows(void* p, int* lo, int* hi) { static_cast<Holder*>(p)->m->chain_logit_rows(*lo, *hi); }
// Feed a prompt token by token through the graph lane; returns the model's next token or -1.
TMCHAIN_API int tmchain_feed(void* p, const int* toks, int n) {
    try { return static_cast<Holder*>(p)->m->gpu_feed(toks, n); }
    catch (const std::exception& e) { g_err = e.what(); return -1; }
}

// A prompt of n >= 3 tokens through the batched layer stack (last token through the decode lane); returns the model's next token or -1.
TMCHAIN_API int tmchain_prefill(void* p, const int* toks, int n) {
    try { return static_cast<Holder*>(p)->m->gpu_prefill(toks, n); }
    catch (const std::exception& e) { g_err = e.what(); return -1; }
}
TMCHAIN_API int tmchain_prefill_prepare(void* p, int max_tokens) {
    try { static_cast<Holder*>(p)->m->gpu_prefill_prepare(max_tokens); return 1; }
    catch (const std::exception& e) { g_err = e.what(); return 0; }
}
TMCHAIN_API double tmchain_prefill_gpu_ms(void* p) { return static_cast<Holder*>(p)->m->last_prefill_gpu_ms(); }

// ---- .tmq containers (include/tmq_reader.h) ---------------------------------------------------------------
// Open a container, make the named tensors resident under one weight handle with aligned offsets, and keep the
// mapping alive (registrations are keyed by addresses inside it). Returns the handle (>= 1000) or -1; fills, per
// tensor, the byte offset inside the handle, the dtype and the number of blocks.
TMCHAIN_API int tmq_upload(const char* path, const char* const* names, int n, unsigned long long* woff, unsigned* dtype,
                           unsigned long long* nblocks) {
    try {
        static std::vector<std::unique_ptr<tmmq::Mapped>> keep;
        auto m = std::make_unique<tmmq::Mapped>();
        if (!m->open(path)) { g_err = std::string("tmq: cannot open or parse ") + path; return -1; }
        std::vector<std::string> nm(names, names + n);
        std::vector<std::uint64_t> off;
        std::vector<std::uint32_t> dts;                    // the dtype each tensor has on the device (GGUF Q4_0 becomes Q4_0)
        const int id = tmmq::upload_tensors(*m, nm, &off, &dts);
        for (int i = 0; i < n; ++i) {
            const tmmq::TensorInfo* t = m->find(nm[(size_t)i]);
            woff[i] = off[(size_t)i]; dtype[i] = dts[(size_t)i]; nblocks[i] = t->nblocks;
        }
        keep.push_back(std::move(m));
        return id;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}
