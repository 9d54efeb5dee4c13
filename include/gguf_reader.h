// include/gguf_reader.h — tensor index of a GGUF v3 file, read in place from a mapping.
//
// What the reference's tensormark/gguf_native.h:142-222 (parse_gguf_index) gives its container reader
// (tensormark/tmq.h:434-463): for every tensor its name in the engine's naming, its GGUF type, its shape outermost
// first, the absolute byte offset of its payload and its block count - or a refusal of the whole file. Written from
// the published GGUF layout:
//
//   "GGUF" | u32 version | u64 tensor_count | u64 kv_count
//   kv_count x ( string key | u32 value_type | value )         string = u64 length + bytes
//   tensor_count x ( string name | u32 n_dims | n_dims x u64 dims (innermost first) | u32 type | u64 offset )
//   padding to general.alignment (default 32) | tensor data; offsets are relative to its start
//
// Accepted, as the reference accepts: version 3 only; keys and tensor names unique; general.alignment a power of two
// up to 1 MiB; 1 to 4 non-zero dimensions whose product fits 64 bits; the types the engine can read (F32, F16, BF16,
// Q4_0, Q4_1, Q8_0, Q4_K, Q5_K, Q6_K); rows of whole blocks; offsets that are multiples of the alignment; payloads
// that lie inside the file and do not overlap. Anything else refuses the file. Nothing here touches the GPU.
#pragma once

#include <algorithm>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <set>
#include <string>
#include <utility>
#include <vector>

namespace tmgguf {

struct Tensor {
    std::string name;                    // the engine's name when the GGUF name is a known one, else the GGUF name
    std::string gguf_name;
    std::uint32_t gguf_type = 0;         // GGUF's numbering, not the container's
    std::vector<std::uint32_t> shape;    // outermost first
    std::size_t payload = 0;             // absolute byte offset in the file
    std::size_t bytes = 0;
    std::uint64_t nblocks = 0;
};

// Values per block and bytes per block of a GGUF tensor type; false for types outside the engine's set.
inline bool type_geometry(std::uint32_t type, std::uint32_t& elems, std::uint32_t& bytes) {
    switch (type) {
        case 0: elems = 1; bytes = 4; return true;        // F32
        case 1: case 30: elems = 1; bytes = 2; return true;   // F16, BF16
        case 2: elems = 32; bytes = 18; return true;      // Q4_0, split nibbles
        case 3: elems = 32; bytes = 20; return true;      // Q4_1
        case 8: elems = 32; bytes = 34; return true;      // Q8_0
        case 12: elems = 256; bytes = 144; return true;   // Q4_K
        case 13: elems = 256; bytes = 176; return true;   // Q5_K
        case 14: elems = 256; bytes = 210; return true;   // Q6_K
        default: return false;
    }
}

// Container dtype id (tensormark/tmq.h:48-60) of a GGUF type, as the reference's reader maps them (tmq.h:446-457);
// UINT32_MAX for a type it does not carry. GGUF's Q4_0 becomes dtype 9, NOT the container's own Q4_0 (dtype 1).
inline std::uint32_t container_dtype(std::uint32_t gguf_type) {
    switch (gguf_type) {
        case 0: return 2; case 1: return 3; case 2: return 9; case 3: return 4; case 8: return 0;
        case 12: return 8; case 13: return 5; case 14: return 6; case 30: return 10;
        default: return UINT32_MAX;
    }
}

// GGUF tensor name -> the engine's name for the tensors of a dense Llama-style model (the table the reference keeps
// in gguf_native.h:107-131 and convert_gguf.cpp's map_name); other names are returned unchanged.
inline std::string engine_name(const std::string& g) {
    if (g == "token_embd.weight") return "model.embed_tokens.weight";
    if (g == "output.weight") return "lm_head.weight";
    if (g == "output_norm.weight") return "model.norm.weight";
    if (g.rfind("blk.", 0) != 0) return g;
    const std::size_t dot = g.find('.', 4);
    if (dot == std::string::npos) return g;
    static const std::pair<const char*, const char*> table[] = {
        {"attn_norm.weight", "input_layernorm.weight"},   {"ffn_norm.weight", "post_attention_layernorm.weight"},
        {"attn_q.weight", "self_attn.q_proj.weight"},     {"attn_k.weight", "self_attn.k_proj.weight"},
        {"attn_v.weight", "self_attn.v_proj.weight"},     {"attn_output.weight", "self_attn.o_proj.weight"},
        {"attn_q.bias", "self_attn.q_proj.bias"},         {"attn_k.bias", "self_attn.k_proj.bias"},
        {"attn_v.bias", "self_attn.v_proj.bias"},         {"ffn_gate.weight", "mlp.gate_proj.weight"},
        {"ffn_up.weight", "mlp.up_proj.weight"},          {"ffn_down.weight", "mlp.down_proj.weight"},
    };
    const std::string rest = g.substr(dot + 1);
    for (const auto& [from, to] : table)
        if (rest == from) return "model.layers." + g.substr(4, dot - 4) + "." + to;
    return g;
}

namespace detail {
// Forward-only view of the file; every read checks what is left and latches failure.
class Cursor {
public:
    Cursor(const std::uint8_t* p, std::size_t n) : p_(p), n_(n) {}
    bool ok() const { return ok_; }
    std::size_t at() const { return at_; }
    std::size_t left() const { return n_ - at_; }
    void fail() { ok_ = false; }
    void advance(std::size_t n) { if (!ok_ || n > left()) ok_ = false; else at_ += n; }
    std::uint64_t le(unsigned bytes) {                  // little-endian unsigned of 1..8 bytes
        if (!ok_ || bytes > left()) { ok_ = false; return 0; }
        std::uint64_t v = 0;
        for (unsigned i = 0; i < bytes; ++i) v |= (std::uint64_t)p_[at_ + i] << (8 * i);
        at_ += bytes;
        return v;
    }
    std::string text() {                                // u64 length + bytes; at most 16 MiB
        const std::uint64_t len = le(8);
        if (!ok_ || len > (1u << 24) || len > left()) { ok_ = false; return {}; }
        std::string s(reinterpret_cast<const char*>(p_ + at_), (std::size_t)len);
        at_ += (std::size_t)len;
        return s;
    }
private:
    const std::uint8_t* p_;
    std::size_t n_, at_ = 0;
    bool ok_ = true;
};

inline unsigned scalar_width(std::uint32_t type) {      // bytes of a fixed-width metadata value, 0 when not one
    switch (type) {
        case 0: case 1: case 7: return 1;
        case 2: case 3: return 2;
        case 4: case 5: case 6: return 4;
        case 10: case 11: case 12: return 8;
        default: return 0;
    }
}
inline void skip_value(Cursor& c, std::uint32_t type, unsigned depth) {
    if (depth > 64) { c.fail(); return; }
    if (const unsigned w = scalar_width(type)) { c.advance(w); return; }
    if (type == 8) { (void)c.text(); return; }
    if (type != 9) { c.fail(); return; }
    const std::uint32_t elem = (std::uint32_t)c.le(4);
    const std::uint64_t count = c.le(8);
    if (!c.ok() || elem > 12) { c.fail(); return; }
    const unsigned w = scalar_width(elem);
    const std::size_t least = w ? w : (elem == 8 ? 8 : 12);        // a string is at least its length, an array its header
    if (count > c.left() / least) { c.fail(); return; }
    if (w) { c.advance((std::size_t)count * w); return; }
    for (std::uint64_t i = 0; i < count && c.ok(); ++i) skip_value(c, elem, depth + 1);
}
}  // namespace detail

// The index of a GGUF file that lies at [data, data + size). On false, `out` and `architecture` are empty.
inline bool parse_index(const std::uint8_t* data, std::size_t size, std::vector<Tensor>& out, std::string& architecture) {
    out.clear();
    architecture.clear();
    if (!data || size < 24 || std::memcmp(data, "GGUF", 4) != 0) return false;
    detail::Cursor c(data, size);
    c.advance(4);
    const std::uint64_t version = c.le(4), ntensors = c.le(8), nkv = c.le(8);
    if (!c.ok() || version != 3 || ntensors > c.left() / 32 || nkv > c.left() / 13) return false;
    std::uint64_t alignment = 32;
    std::string arch;
    std::set<std::string> keys;
    for (std::uint64_t i = 0; i < nkv; ++i) {
        const std::string key = c.text();
        const std::uint32_t type = (std::uint32_t)c.le(4);
        if (!c.ok() || !keys.insert(key).second) return false;
        if (key == "general.architecture") {
            if (type != 8) return false;
            arch = c.text();
        } else if (key == "general.alignment") {
            if (type != 4) return false;
            alignment = c.le(4);
            if (alignment == 0 || alignment > (1u << 20) || (alignment & (alignment - 1))) return false;
        } else {
            detail::skip_value(c, type, 0);
        }
        if (!c.ok()) return false;
    }
    struct Pending { Tensor t; std::uint64_t rel; };
    std::vector<Pending> pend;
    std::set<std::string> names;
    for (std::uint64_t i = 0; i < ntensors; ++i) {
        Pending p;
        p.t.gguf_name = c.text();
        const std::uint64_t rank = c.le(4);
        if (!c.ok() || p.t.gguf_name.empty() || !names.insert(p.t.gguf_name).second || rank == 0 || rank > 4) return false;
        std::uint64_t total = 1, innermost = 0;
        for (std::uint64_t j = 0; j < rank; ++j) {
            const std::uint64_t d = c.le(8);
            if (!c.ok() || d == 0 || d > UINT32_MAX || total > UINT64_MAX / d) return false;
            if (j == 0) innermost = d;
            total *= d;
            p.t.shape.push_back((std::uint32_t)d);
        }
        p.t.gguf_type = (std::uint32_t)c.le(4);
        p.rel = c.le(8);
        std::uint32_t be = 0, bb = 0;
        if (!c.ok() || !type_geometry(p.t.gguf_type, be, bb) || innermost % be || p.rel % alignment) return false;
        p.t.nblocks = total / be;
        if (p.t.nblocks > SIZE_MAX / bb) return false;
        p.t.bytes = (std::size_t)p.t.nblocks * bb;
        std::reverse(p.t.shape.begin(), p.t.shape.end());          // GGUF lists the innermost dimension first
        pend.push_back(std::move(p));
    }
    c.advance((std::size_t)((alignment - c.at() % alignment) % alignment));
    if (!c.ok()) return false;
    const std::size_t data_start = c.at();
    std::set<std::string> mapped;
    std::vector<std::pair<std::size_t, std::size_t>> spans;
    for (Pending& p : pend) {
        if (p.rel > size - data_start || p.t.bytes > size - data_start - (std::size_t)p.rel) return false;
        p.t.payload = data_start + (std::size_t)p.rel;
        p.t.name = engine_name(p.t.gguf_name);
        if (!mapped.insert(p.t.name).second) return false;
        spans.emplace_back(p.t.payload, p.t.payload + p.t.bytes);
    }
    std::sort(spans.begin(), spans.end());
    for (std::size_t i = 1; i < spans.size(); ++i)
        if (spans[i].first < spans[i - 1].second) return false;
    for (Pending& p : pend) out.push_back(std::move(p.t));
    architecture = std::move(arch);
    return true;
}

}  // namespace tmgguf
