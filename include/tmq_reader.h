// include/tmq_reader.h — reader of the .tmq weight container, and its bridge to the CUDA token lane.
//
// Mirror of the container half of the reference's tensormark/tmq.h: the dtype geometry (83-133), the
// record type and THE index parser both of its readers share (136-238, same accept / reject rules) and
// the mmap-backed reader `Mapped` (248-463) reduced to what the matmul path needs: open, the tensor
// table, find. A file that starts with "GGUF" is read natively (tmq.h:434-463): its index comes from
// include/gguf_reader.h, GGUF types map to container dtypes (GGUF's Q4_0 to dtype 9, whose nibble order differs
// from the container's Q4_0), and only the text model's tensors are kept (embedding, head, final norm, layers).
// Wiring policy (mlock, TM_RESIDENT) and the demand-paged reader are outside this path.
//
// File format ("TMQ1"): u32 tensor count, then per tensor
//   u32 name_len | name | u32 dtype | u32 ndims | ndims x u32 shape | u64 nblocks | nblocks blocks
// with no padding between records and nothing after the last one. Payloads therefore lie at arbitrary
// byte offsets; upload_tensors() below packs them into one device buffer at aligned offsets
// (tm_cuda_tok_wbuf_pack), which is what the streaming GEMV needs and what lets tensors of one layer
// share a weight handle.
#pragma once

#include "cuda_shim.h"
#include "gguf_reader.h"
#include "quant.h"

#include <cstddef>
#include <cstdint>
#include <cstring>
#include <limits>
#include <map>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace tmmq {

// Serialized dtype ids of the container (tensormark/tmq.h:48-60).
enum class Dtype : std::uint32_t { Q8_0 = 0, Q4_0 = 1, F32 = 2, F16 = 3, Q4_1 = 4, Q5_K = 5, Q6_K = 6, TQ2 = 7, Q4_K = 8, GGUF_Q4_0 = 9, BF16 = 10 };

// The ids a .tmq record may carry (tmq.h:63-65: up to TQ2; 8..10 only come from the GGUF-native reader).
inline constexpr bool known_dtype(std::uint32_t id) { return id <= 7u; }

inline constexpr std::uint32_t block_elems(std::uint32_t dtype) {
    switch (dtype) {
        case 0: case 1: case 4: case 9: return 32;
        case 2: case 3: case 10: return 1;
        case 5: case 6: case 8: return 256;
        case 7: return 128;
        default: return 0;
    }
}
inline constexpr std::size_t block_bytes(std::uint32_t dtype) {
    switch (dtype) {
        case 0: return 34; case 1: return 18; case 2: return 4; case 3: return 2; case 4: return 20;
        case 5: return 176; case 6: return 210; case 7: return 34; case 8: return 144; case 9: return 18; case 10: return 2;
        default: return 0;
    }
}
inline constexpr std::size_t weight_bytes(Dtype dtype, std::size_t out, std::size_t in) {
    const std::uint32_t id = static_cast<std::uint32_t>(dtype);
    const std::size_t e = block_elems(id);
    return (e == 0 || in % e != 0) ? 0 : out * (in / e) * block_bytes(id);
}

struct TmqRecord {
    std::string name;
    std::uint32_t dtype = 0;
    std::vector<std::uint32_t> shape;
    std::uint64_t nblocks = 0;
    std::size_t payload = 0;      // byte offset of the first block in the file
    std::size_t length = 0;       // payload bytes
};

// The index parser (tmq.h:162-238). `fill(dst, n, at)` copies n bytes from file offset `at`; it is only called
// for ranges that lie inside the file. Accepted: known dtypes, rank >= 1 bounded by the bytes left, names of at
// most 1 MiB, no zero dimension, nblocks == product(shape) / block_elems, payload inside the file, and the
// last record ending exactly at the end of the file. Everything else is rejected.
template <class Fill>
[[nodiscard]] inline bool parse_tmq_index(std::size_t file_size, const Fill& fill, std::vector<TmqRecord>& out) {
    if (file_size < 8) return false;
    std::size_t at = 0;
    const auto left = [&]() { return file_size - at; };
    const auto take = [&](void* dst, std::size_t n) {
        if (n > left()) return false;
        if (n && !fill(dst, n, at)) return false;
        at += n;
        return true;
    };
    char magic[4];
    std::uint32_t count = 0;
    if (!take(magic, 4) || std::memcmp(magic, "TMQ1", 4) != 0 || !take(&count, 4)) return false;
    constexpr std::size_t kSmallestRecord = 4 + 4 + 4 + 4 + 8 + 2;      // empty name, rank 1, one F16 value
    if (count > left() / kSmallestRecord) return false;
    out.clear();
    out.reserve(count);
    for (std::uint32_t i = 0; i < count; ++i) {
        TmqRecord r;
        std::uint32_t name_len = 0, rank = 0;
        if (!take(&name_len, 4) || name_len > (1u << 20) || name_len > left()) return false;
        r.name.resize(name_len);
        if (!take(r.name.data(), name_len)) return false;
        if (!take(&r.dtype, 4) || !known_dtype(r.dtype)) return false;
        if (!take(&rank, 4) || rank == 0 || left() < 8 || rank > (left() - 8) / 4) return false;
        r.shape.resize(rank);
        std::uint64_t n = 1;
        for (std::uint32_t& d : r.shape) {
            if (!take(&d, 4) || d == 0 || n > std::numeric_limits<std::uint64_t>::max() / d) return false;
            n *= d;
        }
        if (!take(&r.nblocks, 8)) return false;
        const std::uint32_t be = block_elems(r.dtype);
        const std::size_t bb = block_bytes(r.dtype);
        if (!be || !bb || n % be != 0 || r.nblocks != n / be || r.nblocks > left() / bb) return false;
        r.payload = at;
        r.length = static_cast<std::size_t>(r.nblocks) * bb;
        at += r.length;
        out.push_back(std::move(r));
    }
    return at == file_size;
}

struct TensorInfo {
    std::uint32_t dtype = 0;
    std::vector<std::uint32_t> shape;
    const std::uint8_t* blocks = nullptr;         // view into the mapping
    std::uint64_t nblocks = 0;
    std::size_t bytes = 0;
    std::uint64_t n() const { std::uint64_t v = 1; for (auto d : shape) v *= d; return v; }
};

// Read-only mapping of one container file with its tensor table.
class Mapped {
public:
    Mapped() = default;
    Mapped(const Mapped&) = delete;
    Mapped& operator=(const Mapped&) = delete;
    ~Mapped() { close(); }

    // false (and the previous state kept) when the file cannot be opened, mapped or parsed
    [[nodiscard]] bool open(const std::string& path) {
        const int fd = ::open(path.c_str(), O_RDONLY);
        if (fd < 0) return false;
        struct stat sb;
        if (::fstat(fd, &sb) != 0 || sb.st_size < 8) { ::close(fd); return false; }
        const std::size_t size = static_cast<std::size_t>(sb.st_size);
        void* p = ::mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
        ::close(fd);
        if (p == MAP_FAILED) return false;
        const std::uint8_t* base = static_cast<const std::uint8_t*>(p);
        std::map<std::string, TensorInfo> table;
        std::string arch;
        if (std::memcmp(base, "GGUF", 4) == 0) {
            std::vector<tmgguf::Tensor> idx;
            if (!tmgguf::parse_index(base, size, idx, arch)) { ::munmap(p, size); return false; }
            for (tmgguf::Tensor& g : idx) {
                // the text model only; a vision tower or an unknown tensor is never given an engine name (tmq.h:439-445)
                const bool keep = g.name == "model.embed_tokens.weight" || g.name == "lm_head.weight" || g.name == "model.norm.weight" ||
                                  g.name.rfind("model.layers.", 0) == 0;
                if (!keep) continue;
                TensorInfo t;
                t.dtype = tmgguf::container_dtype(g.gguf_type);
                if (t.dtype == UINT32_MAX) { ::munmap(p, size); return false; }
                t.shape = std::move(g.shape); t.blocks = base + g.payload; t.nblocks = g.nblocks; t.bytes = g.bytes;
                if (!table.emplace(std::move(g.name), std::move(t)).second) { ::munmap(p, size); return false; }
            }
        } else {
            std::vector<TmqRecord> recs;
            const bool ok = parse_tmq_index(size, [&](void* dst, std::size_t n, std::size_t at) { std::memcpy(dst, base + at, n); return true; }, recs);
            if (!ok) { ::munmap(p, size); return false; }
            for (TmqRecord& r : recs) {
                TensorInfo t;
                t.dtype = r.dtype; t.shape = std::move(r.shape); t.blocks = base + r.payload; t.nblocks = r.nblocks; t.bytes = r.length;
                table[std::move(r.name)] = std::move(t);
            }
        }
        close();
        base_ = base; size_ = size; tensors_ = std::move(table); architecture_ = std::move(arch);
        return true;
    }
    void close() {
        if (base_) ::munmap(const_cast<std::uint8_t*>(base_), size_);
        base_ = nullptr; size_ = 0; tensors_.clear(); architecture_.clear();
    }
    const std::string& architecture() const { return architecture_; }      // general.architecture of a GGUF file, "" for .tmq
    const std::uint8_t* base() const { return base_; }
    std::size_t size() const { return size_; }
    const std::map<std::string, TensorInfo>& tensors() const { return tensors_; }
    const TensorInfo* find(const std::string& name) const {
        const auto it = tensors_.find(name);
        return it == tensors_.end() ? nullptr : &it->second;
    }

private:
    const std::uint8_t* base_ = nullptr;
    std::size_t size_ = 0;
    std::map<std::string, TensorInfo> tensors_;
    std::string architecture_;
};

// Make the named tensors resident on the GPU as ONE weight handle with aligned offsets. Afterwards the lane's
// tm_cuda_tok_wbuf(tensor.blocks, ...) (and so tmllama::CudaLlama, which registers by pointer) finds them there.
// Tensors in GGUF's own Q4_0 (dtype 9) are reordered on the device into the container's Q4_0 (the converter's nibble
// reorder, tensormark/convert_gguf.cpp:124-135, bit-identical weights): `dtypes`, when given, receives the dtype each
// tensor has ON THE DEVICE (1 for those). Throws std::invalid_argument for an unknown name, std::runtime_error when
// the upload fails.
inline int upload_tensors(const Mapped& file, const std::vector<std::string>& names, std::vector<std::uint64_t>* offsets = nullptr,
                          std::vector<std::uint32_t>* dtypes = nullptr) {
    std::vector<const void*> ptrs;
    std::vector<std::size_t> bytes;
    for (const std::string& nm : names) {
        const TensorInfo* t = file.find(nm);
        if (!t) throw std::invalid_argument("tmq: no tensor named " + nm);
        ptrs.push_back(t->blocks);
        bytes.push_back(t->bytes);
    }
    std::vector<std::uint64_t> woff(names.size());
    const int id = tm_cuda_tok_wbuf_pack(ptrs.data(), bytes.data(), static_cast<unsigned>(ptrs.size()), woff.data());
    if (id < 0) throw std::runtime_error(std::string("tmq: upload failed: ") + tm_cuda_last_error());
    if (dtypes) dtypes->clear();
    for (std::size_t i = 0; i < names.size(); ++i) {
        const TensorInfo* t = file.find(names[i]);
        std::uint32_t dt = t->dtype;
        if (dt == static_cast<std::uint32_t>(Dtype::GGUF_Q4_0)) {
            if (!tm_cuda_tok_wbuf_q4_from_gguf(id, woff[i], static_cast<std::size_t>(t->nblocks)))
                throw std::runtime_error(std::string("tmq: Q4_0 reorder failed: ") + tm_cuda_last_error());
            dt = static_cast<std::uint32_t>(Dtype::Q4_0);
        }
        if (dtypes) dtypes->push_back(dt);
    }
    if (offsets) *offsets = std::move(woff);
    return id;
}

}  // namespace tmmq
