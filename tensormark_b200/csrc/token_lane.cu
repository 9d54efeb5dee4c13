// token_lane.cu — the per-token decode lane of the C ABI.
//
// CUDA counterpart of the reference's "gpu2" token pipeline (tensormark/metal.h:
// 2236-2300 slots, 3074-3190 begin/flush/end/async, 3282-3337 weight handles,
// 3457-3765 GEMV and elementwise encoders, 3913-4275 rope table, K/V cache and
// attention), behind the same entry points (tensormark/metal_shim.mm:22-152).
//
// Where Metal encodes dispatches into a command buffer and commits it, this lane
// launches kernels on one CUDA stream: encode order is execution order, tok_end is
// a stream synchronisation, tok_end_async records an event. Slots are device
// buffers; weights are copied into device memory once per tensor (or once per
// mapping for the zero-copy form) and addressed as (handle, byte offset).
//
// The void encoders cannot return an error. A bad argument latches a sticky
// failure instead of throwing across the C boundary: nothing is launched for that
// call and the next tok_end / tok_flush / tok_wait_pending returns false.
#include "cuda_shim.h"
#include "common.cuh"
#include "glue.h"
#include "state.h"

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

namespace tmc {

namespace {

constexpr int kMaxSlots = 4096;          // plain slots are ids below the first weight handle
constexpr int kFirstWeight = 1000;

void latch(const char* fmt, ...) {
    char buf[400];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    fail("%s", buf);
    state().sticky = true;
}

// Device pointer of a slot that must already hold `bytes`; nullptr (and a latched
// error) otherwise. A slot may be created, but not grown, while a token is encoded.
uint8_t* slot_ptr(int sid, size_t bytes, const char* who) {
    State& s = state();
    if (sid < 0 || sid >= kFirstWeight) { latch("%s: slot id %d out of range", who, sid); return nullptr; }
    if ((int)s.slots.size() <= sid) s.slots.resize((size_t)sid + 1);
    Slot& sl = s.slots[sid];
    if (sl.ptr && sl.bytes >= bytes) return sl.ptr;
    if (sl.shared) { latch("%s: shared slot %d holds %zu bytes, %zu wanted", who, sid, sl.bytes, bytes); return nullptr; }
    if (sl.ptr && s.encoding) { latch("%s: slot %d must be reserved before token encoding (%zu > %zu bytes)", who, sid, bytes, sl.bytes); return nullptr; }
    if (bytes == 0) { latch("%s: slot %d is empty", who, sid); return nullptr; }
    uint8_t* p = nullptr;
    const size_t want = (bytes + 255) / 256 * 256;
    if (cudaMalloc(&p, want) != cudaSuccess) { cudaGetLastError(); latch("%s: slot %d allocation of %zu bytes failed", who, sid, want); return nullptr; }
    cudaMemsetAsync(p, 0, want, s.stream);
    if (sl.ptr) {
        cudaMemcpyAsync(p, sl.ptr, sl.bytes, cudaMemcpyDeviceToDevice, s.stream);
        cudaStreamSynchronize(s.stream);
        cudaFree(sl.ptr);
    }
    sl.ptr = p; sl.bytes = want;
    return p;
}

const uint8_t* weight_ptr(int wid, uint64_t woff, size_t bytes, const char* who) {
    State& s = state();
    const int i = wid - kFirstWeight;
    if (i < 0 || i >= (int)s.wbufs.size() || !s.wbufs[i].ptr) { latch("%s: unknown weight handle %d", who, wid); return nullptr; }
    if (woff > s.wbufs[i].bytes || bytes > s.wbufs[i].bytes - woff) { latch("%s: weight range [%llu, +%zu) outside handle %d (%zu bytes)", who, (unsigned long long)woff, bytes, wid, s.wbufs[i].bytes); return nullptr; }
    return s.wbufs[i].ptr + woff;
}

// (cos, sin) table, built on the host with the reference's expression
// (metal.h:3926-3941: inv = pow(theta, -2j/dh) in fp32, angle = (float)p * inv).
// Grows geometrically; a rebuild waits for the lane so no kernel reads a freed table.
bool ensure_rope(unsigned dh, unsigned need, float theta) {
    State& s = state();
    if (!dh || (dh & 1u)) { latch("rope: odd head dim %u", dh); return false; }
    if (!need) need = 1;
    const bool same = s.rope_tbl && s.rope_dh == dh && s.rope_theta == theta;
    if (same && s.rope_cap >= need) return true;
    unsigned cap = same ? s.rope_cap : 0;
    while (cap < need) cap = cap ? cap * 2 : 64;
    const unsigned half = dh / 2;
    std::vector<float> tbl((size_t)cap * half * 2);
    for (unsigned j = 0; j < half; ++j) {
        const float inv = std::pow(theta, -2.0f * (float)j / (float)dh);
        for (unsigned p = 0; p < cap; ++p) {
            const float ang = (float)p * inv;
            tbl[2 * ((size_t)p * half + j)] = std::cos(ang);
            tbl[2 * ((size_t)p * half + j) + 1] = std::sin(ang);
        }
    }
    float* d = nullptr;
    if (cudaMalloc(&d, tbl.size() * 4) != cudaSuccess) { cudaGetLastError(); latch("rope: table allocation failed"); return false; }
    cudaStreamSynchronize(s.stream);
    cudaMemcpy(d, tbl.data(), tbl.size() * 4, cudaMemcpyHostToDevice);
    if (s.rope_tbl) cudaFree(s.rope_tbl);
    s.rope_tbl = d; s.rope_dh = dh; s.rope_cap = cap; s.rope_theta = theta;
    return true;
}

size_t kv_elem() { return state().kv_half ? 2 : 4; }

bool finish(const char* where) {
    State& s = state();
    const bool ok = sync_stream(s.stream, where);
    const bool sticky = s.sticky;
    s.sticky = false;
    s.encoding = false;
    if (sticky) { ++s.fallbacks; return false; }
    return ok;
}

unsigned long long* choose_scratch() {
    static unsigned long long* p = nullptr;
    if (!p) {
        if (cudaMalloc(&p, 16) != cudaSuccess) { cudaGetLastError(); p = nullptr; return nullptr; }
        cudaMemset(p, 0, 16);
    }
    return p;
}

void gemv_common(int xslot, int wid, int yslot, size_t yoff, unsigned N, unsigned K, unsigned dtype,
                 const uint64_t* seg_woff, const unsigned* seg_rows, unsigned nseg, const char* who) {
    State& s = state();
    if (!ensure_init(-1)) { s.sticky = true; return; }
    const size_t row_bytes = weight_bytes(dtype, 1, K);
    if (!row_bytes) { latch("%s: K=%u is not whole blocks of dtype %u", who, K, dtype); return; }
    if (yoff % 4) { latch("%s: output byte offset %zu is not a multiple of 4", who, yoff); return; }
    SegTable t;
    if (!make_segments(t, N, seg_woff, seg_rows, nseg)) { s.sticky = true; return; }
    // all segments live in the handle's buffer: express them relative to its base
    const int i = wid - kFirstWeight;
    if (i < 0 || i >= (int)s.wbufs.size() || !s.wbufs[i].ptr) { latch("%s: unknown weight handle %d", who, wid); return; }
    for (unsigned k = 0; k < nseg; ++k)
        if (t.woff[k] > s.wbufs[i].bytes || (size_t)seg_rows[k] * row_bytes > s.wbufs[i].bytes - t.woff[k]) {
            latch("%s: segment %u lies outside weight handle %d", who, k, wid); return;
        }
    const float* x = (const float*)slot_ptr(xslot, (size_t)K * 4, who);
    uint8_t* y = slot_ptr(yslot, yoff + (size_t)N * 4, who);
    if (!x || !y) return;
    if (!launch_gemv(x, s.wbufs[i].ptr, (float*)(y + yoff), N, K, dtype, t, s.stream)) s.sticky = true;
}

}  // namespace

// What the prefill layer stack (llama_stack.cu) shares with the lane: the resident weights, the rope table, the slots.
const uint8_t* lane_weight_ptr(int wid, uint64_t woff, size_t bytes) { return weight_ptr(wid, woff, bytes, "llama stack"); }
const float* lane_rope_table(unsigned dh, unsigned need, float theta, unsigned* entries) {
    if (!ensure_rope(dh, need, theta)) return nullptr;
    if (entries) *entries = state().rope_cap * (dh / 2);
    return state().rope_tbl;
}
uint8_t* lane_slot_ptr(int sid, size_t bytes, const char* who) { return slot_ptr(sid, bytes, who); }

}  // namespace tmc

using namespace tmc;

extern "C" {

bool tm_cuda_tok_begin(void) {
    if (!ensure_init(-1)) return false;
    state().encoding = true;
    return true;
}
bool tm_cuda_tok_flush(void) { return ensure_init(-1) && finish("tok_flush"); }
bool tm_cuda_tok_end(int outslot, float* dst, unsigned n) {
    if (!ensure_init(-1)) return false;
    State& s = state();
    if (n) {
        if (!dst) return fail("tok_end: null destination");
        const uint8_t* p = slot_ptr(outslot, (size_t)n * 4, "tok_end");
        if (p && cudaMemcpyAsync(dst, p, (size_t)n * 4, cudaMemcpyDeviceToHost, s.stream) != cudaSuccess) { check_launch("tok_end: download"); s.sticky = true; }
    }
    return finish("tok_end");
}
bool tm_cuda_tok_end_async(void) {
    if (!ensure_init(-1)) return false;
    State& s = state();
    cudaEvent_t ev;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) return check_launch("tok_end_async");
    cudaEventRecord(ev, s.stream);
    s.pending.push_back(ev);
    s.encoding = false;
    return true;
}
bool tm_cuda_tok_wait_pending(void) {
    if (!ensure_init(-1)) return false;
    State& s = state();
    bool ok = true;
    for (cudaEvent_t ev : s.pending) {
        if (cudaEventSynchronize(ev) != cudaSuccess) { ok = false; fail("tok_wait_pending: %s", cudaGetErrorString(cudaGetLastError())); }
        cudaEventDestroy(ev);
    }
    s.pending.clear();
    return finish("tok_wait_pending") && ok;
}
bool tm_cuda_tok_reserve(int slot, size_t bytes) {
    if (!ensure_init(-1)) return false;
    State& s = state();
    if (s.encoding) return fail("tok_reserve: not between tok_begin and the end of the token");
    const bool before = s.sticky;
    const bool ok = slot_ptr(slot, bytes, "tok_reserve") != nullptr;
    if (!ok) s.sticky = before;            // a bool entry reports by its return value
    return ok;
}
bool tm_cuda_tok_upload(int slot, size_t byte_off, const void* src, size_t bytes) {
    if (!ensure_init(-1)) return false;
    State& s = state();
    if (!src && bytes) return fail("tok_upload: null source");
    const bool before = s.sticky;
    uint8_t* p = slot_ptr(slot, byte_off + bytes, "tok_upload");
    if (!p) { s.sticky = before; return false; }
    // Pageable host memory: the copy is staged before the call returns, so the
    // caller may reuse `src` at once; it is still ordered after earlier lane work.
    if (bytes && cudaMemcpyAsync(p + byte_off, src, bytes, cudaMemcpyHostToDevice, s.stream) != cudaSuccess) return check_launch("tok_upload");
    return true;
}
bool tm_cuda_tok_download(int slot, size_t byte_off, void* dst, size_t bytes) {
    if (!ensure_init(-1)) return false;
    State& s = state();
    if (!dst && bytes) return fail("tok_download: null destination");
    const bool before = s.sticky;
    const uint8_t* p = slot_ptr(slot, byte_off + bytes, "tok_download");
    if (!p) { s.sticky = before; return false; }
    if (bytes && cudaMemcpyAsync(dst, p + byte_off, bytes, cudaMemcpyDeviceToHost, s.stream) != cudaSuccess) return check_launch("tok_download");
    return sync_stream(s.stream, "tok_download");
}
bool tm_cuda_tok_kv_reserve(int slot, size_t n) { return ensure_init(-1) && tm_cuda_tok_reserve(slot, n * kv_elem()); }
bool tm_cuda_tok_kv_upload(int slot, size_t elem_off, const float* src, size_t n) {
    if (!ensure_init(-1)) return false;
    State& s = state();
    if (!s.kv_half) return tm_cuda_tok_upload(slot, elem_off * 4, src, n * 4);
    if (!src && n) return fail("tok_kv_upload: null source");
    const bool before = s.sticky;
    uint8_t* p = slot_ptr(slot, (elem_off + n) * 2, "tok_kv_upload");
    if (!p) { s.sticky = before; return false; }
    if (!n) return true;
    float* stage = (float*)s.io_big.get(n * 4);
    if (!stage) return fail("tok_kv_upload: out of device memory");
    if (cudaMemcpyAsync(stage, src, n * 4, cudaMemcpyHostToDevice, s.stream) != cudaSuccess) return check_launch("tok_kv_upload");
    return launch_f32_to_half(stage, p + elem_off * 2, n, s.stream);
}
bool tm_cuda_tok_kv_download(int slot, size_t elem_off, float* dst, size_t n) {
    if (!ensure_init(-1)) return false;
    State& s = state();
    if (!s.kv_half) return tm_cuda_tok_download(slot, elem_off * 4, dst, n * 4);
    if (!dst && n) return fail("tok_kv_download: null destination");
    const bool before = s.sticky;
    const uint8_t* p = slot_ptr(slot, (elem_off + n) * 2, "tok_kv_download");
    if (!p) { s.sticky = before; return false; }
    if (!n) return true;
    float* stage = (float*)s.io_big.get(n * 4);
    if (!stage) return fail("tok_kv_download: out of device memory");
    if (!launch_half_to_f32(p + elem_off * 2, stage, n, s.stream)) return false;
    if (cudaMemcpyAsync(dst, stage, n * 4, cudaMemcpyDeviceToHost, s.stream) != cudaSuccess) return check_launch("tok_kv_download");
    return sync_stream(s.stream, "tok_kv_download");
}

int tm_cuda_tok_wbuf(const void* tensor_ptr, size_t bytes, const void* map_base, size_t map_size, int zero_copy,
                     uint64_t* woff_out) {
    if (woff_out) *woff_out = 0;
    if (!ensure_init(-1) || !tensor_ptr || !bytes || !woff_out) { fail("tok_wbuf: bad arguments"); return -1; }
    State& s = state();
    auto it = s.wreg.find(tensor_ptr);
    if (it != s.wreg.end()) { *woff_out = it->second.second; return it->second.first; }
    if (zero_copy) {
        const uintptr_t base = (uintptr_t)map_base, ptr = (uintptr_t)tensor_ptr;
        if (!base || ptr < base || ptr - base > map_size || bytes > map_size - (ptr - base)) { fail("tok_wbuf: tensor outside the mapping"); return -1; }
        if (s.shared_id < 0 || s.shared_base != map_base) {
            // One resident copy of the whole mapping; tensor offsets are byte offsets into it.
            uint8_t* d = nullptr;
            if (cudaMalloc(&d, map_size + 32) != cudaSuccess) { cudaGetLastError(); fail("tok_wbuf: %zu bytes of device memory unavailable", map_size); return -1; }
            if (cudaMemcpyAsync(d, map_base, map_size, cudaMemcpyHostToDevice, s.stream) != cudaSuccess) { cudaFree(d); check_launch("tok_wbuf: upload"); return -1; }
            cudaMemsetAsync(d + map_size, 0, 32, s.stream);
            s.wbufs.push_back({d, map_size});
            s.shared_id = kFirstWeight + (int)s.wbufs.size() - 1;
            s.shared_base = map_base;
        }
        *woff_out = (uint64_t)(ptr - base);
        s.wreg[tensor_ptr] = {s.shared_id, *woff_out};
        return s.shared_id;
    }
    uint8_t* d = nullptr;
    if (cudaMalloc(&d, bytes + 32) != cudaSuccess) { cudaGetLastError(); fail("tok_wbuf: %zu bytes of device memory unavailable", bytes); return -1; }
    if (cudaMemcpyAsync(d, tensor_ptr, bytes, cudaMemcpyHostToDevice, s.stream) != cudaSuccess) { cudaFree(d); check_launch("tok_wbuf: upload"); return -1; }
    cudaMemsetAsync(d + bytes, 0, 32, s.stream);
    s.wbufs.push_back({d, bytes});
    const int id = kFirstWeight + (int)s.wbufs.size() - 1;
    s.wreg[tensor_ptr] = {id, 0};
    return id;
}

// Several tensors into ONE device buffer, each at a 256-byte aligned offset: the tensors of a container file lie
// at arbitrary byte offsets (records follow one another without padding), which a mirror of the mapping would
// inherit, and the streaming GEMV wants 16-byte aligned rows. One handle for all of them keeps the segmented
// launches (q|k|v, gate|up) possible. Returns the handle, fills woff_out[i]; -1 on failure. Tensors already
// registered keep their old registration and are copied again under the new handle.
int tm_cuda_tok_wbuf_pack(const void* const* tensor_ptrs, const size_t* bytes, unsigned n, uint64_t* woff_out) {
    if (!ensure_init(-1) || !tensor_ptrs || !bytes || !woff_out || n == 0) { fail("tok_wbuf_pack: bad arguments"); return -1; }
    State& s = state();
    size_t total = 0;
    for (unsigned i = 0; i < n; ++i) {
        if (!tensor_ptrs[i] || !bytes[i]) { fail("tok_wbuf_pack: tensor %u is empty", i); return -1; }
        woff_out[i] = total;
        total += (bytes[i] + 32 + 255) / 256 * 256;          // 32 bytes of slack after every tensor, as for single tensors
    }
    uint8_t* d = nullptr;
    if (cudaMalloc(&d, total) != cudaSuccess) { cudaGetLastError(); fail("tok_wbuf_pack: %zu bytes of device memory unavailable", total); return -1; }
    cudaMemsetAsync(d, 0, total, s.stream);
    for (unsigned i = 0; i < n; ++i)
        if (cudaMemcpyAsync(d + woff_out[i], tensor_ptrs[i], bytes[i], cudaMemcpyHostToDevice, s.stream) != cudaSuccess) {
            cudaStreamSynchronize(s.stream); cudaFree(d); check_launch("tok_wbuf_pack: upload"); return -1;
        }
    s.wbufs.push_back({d, total});
    const int id = kFirstWeight + (int)s.wbufs.size() - 1;
    for (unsigned i = 0; i < n; ++i) s.wreg[tensor_ptrs[i]] = {id, woff_out[i]};
    return id;
}

bool tm_cuda_tok_probe_copy(int srcslot, size_t src_off, int dstslot, unsigned n) {
    if (!tm_cuda_tok_begin()) return false;
    State& s = state();
    const uint8_t* src = srcslot >= kFirstWeight ? weight_ptr(srcslot, src_off, n, "tok_probe_copy")
                                                 : slot_ptr(srcslot, src_off + n, "tok_probe_copy");
    if (src && srcslot < kFirstWeight) src += src_off;
    s.encoding = false;                                  // the destination may be created here
    uint8_t* dst = slot_ptr(dstslot, n, "tok_probe_copy");
    s.encoding = true;
    if (src && dst && !launch_copy_bytes(src, dst, n, s.stream)) s.sticky = true;
    return tm_cuda_tok_end(dstslot, nullptr, 0);
}

void tm_cuda_tok_gemv(int xslot, int wid, uint64_t woff, int yslot, size_t yoff, unsigned N, unsigned K) {
    gemv_common(xslot, wid, yslot, yoff, N, K, DT_Q4_0, &woff, &N, 1, "tok_gemv");
}
bool tm_cuda_tok_gemv_seg_supported(unsigned dtype) {
    return dtype == DT_Q8_0 || dtype == DT_Q4_0 || dtype == DT_Q4_1 || dtype == DT_Q5_K || dtype == DT_Q6_K || dtype == DT_Q4_K;
}
void tm_cuda_tok_gemv_seg(int xslot, int wid, int yslot, size_t yoff, unsigned N, unsigned K,
                          const uint64_t* seg_woff, const unsigned* seg_rows, unsigned nseg) {
    gemv_common(xslot, wid, yslot, yoff, N, K, DT_Q4_0, seg_woff, seg_rows, nseg, "tok_gemv_seg");
}
void tm_cuda_tok_gemv_seg_dt(int xslot, int wid, int yslot, size_t yoff, unsigned N, unsigned K, unsigned dtype,
                             const uint64_t* seg_woff, const unsigned* seg_rows, unsigned nseg) {
    if (!tm_cuda_tok_gemv_seg_supported(dtype)) { ensure_init(-1); fail("tok_gemv_seg_dt: no segmented GEMV for dtype %u", dtype); state().sticky = true; return; }
    gemv_common(xslot, wid, yslot, yoff, N, K, dtype, seg_woff, seg_rows, nseg, "tok_gemv_seg_dt");
}
void tm_cuda_tok_gemv_kq(int xslot, int wid, uint64_t woff, int yslot, size_t yoff, unsigned N, unsigned K, unsigned dtype) {
    if (!tm_cuda_tok_gemv_seg_supported(dtype)) { ensure_init(-1); fail("tok_gemv_kq: no GEMV for dtype %u", dtype); state().sticky = true; return; }
    gemv_common(xslot, wid, yslot, yoff, N, K, dtype, &woff, &N, 1, "tok_gemv_kq");
}

void tm_cuda_tok_embed_kq(int tokslot, unsigned idx, int wid, uint64_t woff, int xslot, unsigned D, unsigned dtype) {
    if (!ensure_init(-1)) return;
    State& s = state();
    const unsigned* tok = (const unsigned*)slot_ptr(tokslot, sizeof(unsigned) * ((size_t)idx + 1), "tok_embed");
    float* x = (float*)slot_ptr(xslot, (size_t)D * 4, "tok_embed");
    const uint8_t* W = weight_ptr(wid, woff, 0, "tok_embed");
    if (!tok || !x || !W) return;
    if (!launch_embed_row(tok, idx, W, x, D, dtype, s.stream)) s.sticky = true;
}
void tm_cuda_tok_embed_q4(int tokslot, unsigned idx, int wid, uint64_t woff, int xslot, unsigned D) {
    tm_cuda_tok_embed_kq(tokslot, idx, wid, woff, xslot, D, DT_Q4_0);
}
// F16 tensors (tensormark/metal.h:3693-3721 tok_gemv_h, 3260-3271 tok_embed_h). woff is a byte offset into the handle.
void tm_cuda_tok_gemv_h(int xslot, int wid, uint64_t woff, int yslot, size_t yoff, unsigned N, unsigned K) {
    if (!ensure_init(-1)) return;
    State& s = state();
    if (yoff % 4 || woff % 2) { latch("tok_gemv_h: misaligned offset"); return; }
    const float* x = (const float*)slot_ptr(xslot, (size_t)K * 4, "tok_gemv_h");
    uint8_t* y = slot_ptr(yslot, yoff + (size_t)N * 4, "tok_gemv_h");
    const uint8_t* W = weight_ptr(wid, woff, (size_t)N * K * 2, "tok_gemv_h");
    if (!x || !y || !W) return;
    if (!launch_gemv_half(x, W, (float*)(y + yoff), N, K, false, s.stream)) s.sticky = true;
}
void tm_cuda_tok_embed_h(int tokslot, unsigned idx, int wid, uint64_t woff, int xslot, unsigned D) {
    if (!ensure_init(-1)) return;
    State& s = state();
    const unsigned* tok = (const unsigned*)slot_ptr(tokslot, sizeof(unsigned) * ((size_t)idx + 1), "tok_embed_h");
    float* x = (float*)slot_ptr(xslot, (size_t)D * 4, "tok_embed_h");
    const uint8_t* W = weight_ptr(wid, woff, 0, "tok_embed_h");
    if (!tok || !x || !W) return;
    if (woff % 2) { latch("tok_embed_h: misaligned offset"); return; }
    if (!launch_embed_half(tok, idx, W, x, D, false, s.stream)) s.sticky = true;
}
// The Q4_0 blocks of a registered range arrived in GGUF's split nibble order: rewrite them in place in the container's
// order, after which every Q4_0 kernel serves them (tensormark/convert_gguf.cpp:124-135, done on the device).
bool tm_cuda_tok_wbuf_q4_from_gguf(int wid, uint64_t woff, size_t nblocks) {
    if (!ensure_init(-1)) return false;
    State& s = state();
    if (s.encoding) return fail("tok_wbuf_q4_from_gguf: not while a token is encoded");
    const uint8_t* W = weight_ptr(wid, woff, nblocks * 18, "tok_wbuf_q4_from_gguf");
    if (!W) { s.sticky = false; return false; }
    if (!launch_q4_split_to_interleaved(const_cast<uint8_t*>(W), nblocks, s.stream)) return false;
    return sync_stream(s.stream, "tok_wbuf_q4_from_gguf");
}
void tm_cuda_tok_bias_qkv(int yslot, int biasslot, size_t bias_off, unsigned N) {
    if (!ensure_init(-1)) return;
    State& s = state();
    if (bias_off % 4) { latch("tok_bias_qkv: byte offset %zu is not a multiple of 4", bias_off); return; }
    float* y = (float*)slot_ptr(yslot, (size_t)N * 4, "tok_bias_qkv");
    const uint8_t* b = slot_ptr(biasslot, bias_off + (size_t)N * 4, "tok_bias_qkv");
    if (!y || !b) return;
    if (!launch_bias(y, (const float*)(b + bias_off), N, s.stream)) s.sticky = true;
}
void tm_cuda_tok_rmsnorm(int xslot, const void* w, int outslot, unsigned D, float eps) {
    if (!ensure_init(-1)) return;
    State& s = state();
    if (!w || !D) { latch("tok_rmsnorm: bad arguments"); return; }
    float* dw = nullptr;
    auto it = s.norm_w.find(w);
    if (it != s.norm_w.end()) dw = it->second;
    else {
        // copied once and cached by host pointer, like the reference (metal.h:3725-3735)
        if (cudaMalloc(&dw, (size_t)D * 4) != cudaSuccess) { cudaGetLastError(); latch("tok_rmsnorm: weight allocation failed"); return; }
        cudaMemcpyAsync(dw, w, (size_t)D * 4, cudaMemcpyHostToDevice, s.stream);
        s.norm_w[w] = dw;
    }
    const float* x = (const float*)slot_ptr(xslot, (size_t)D * 4, "tok_rmsnorm");
    float* out = (float*)slot_ptr(outslot, (size_t)D * 4, "tok_rmsnorm");
    if (!x || !out) return;
    if (!launch_rmsnorm(x, dw, out, D, eps, s.stream)) s.sticky = true;
}
void tm_cuda_tok_add(int a, int b, unsigned n) {
    if (!ensure_init(-1)) return;
    State& s = state();
    float* pa = (float*)slot_ptr(a, (size_t)n * 4, "tok_add");
    const float* pb = (const float*)slot_ptr(b, (size_t)n * 4, "tok_add");
    if (!pa || !pb) return;
    if (!launch_add(pa, pb, n, s.stream)) s.sticky = true;
}
void tm_cuda_tok_silu_mul(int g, size_t goff, int u, size_t uoff, unsigned n) {
    if (!ensure_init(-1)) return;
    State& s = state();
    if (goff % 4 || uoff % 4) { latch("tok_silu_mul: byte offsets must be multiples of 4"); return; }
    uint8_t* pg = slot_ptr(g, goff + (size_t)n * 4, "tok_silu_mul");
    const uint8_t* pu = slot_ptr(u, uoff + (size_t)n * 4, "tok_silu_mul");
    if (!pg || !pu) return;
    if (!launch_silu_mul((float*)(pg + goff), (const float*)(pu + uoff), n, s.stream)) s.sticky = true;
}
void tm_cuda_tok_rope_q(int qslot, unsigned H, unsigned dh, int pos, float theta) {
    if (!ensure_init(-1)) return;
    State& s = state();
    if (!ensure_rope(dh, (unsigned)(pos > 0 ? pos + 1 : 1), theta)) return;
    float* q = (float*)slot_ptr(qslot, (size_t)H * dh * 4, "tok_rope_q");
    if (!q) return;
    if (!launch_rope(q, H, dh, pos, s.rope_tbl, s.rope_cap * (dh / 2), s.stream)) s.sticky = true;
}
void tm_cuda_tok_rope_k_cache(int ksrcslot, size_t ksrc_off, int cacheslot, unsigned KVH, unsigned dh, unsigned ctx,
                              int pos, float theta) {
    if (!ensure_init(-1)) return;
    State& s = state();
    if (ksrc_off % 4) { latch("tok_rope_k_cache: byte offset must be a multiple of 4"); return; }
    if (pos < 0 || (unsigned)pos >= ctx) { latch("tok_rope_k_cache: position %d outside the %u-row cache", pos, ctx); return; }
    if (!ensure_rope(dh, ctx, theta)) return;
    const uint8_t* k = slot_ptr(ksrcslot, ksrc_off + (size_t)KVH * dh * 4, "tok_rope_k_cache");
    uint8_t* c = slot_ptr(cacheslot, kv_elem() * KVH * ctx * dh, "tok_rope_k_cache");
    if (!k || !c) return;
    if (!launch_rope_k_cache((const float*)(k + ksrc_off), c, s.kv_half, KVH, dh, ctx, pos, s.rope_tbl, s.rope_cap * (dh / 2), s.stream)) s.sticky = true;
}
void tm_cuda_tok_v_cache(int vsrcslot, size_t vsrc_off, int cacheslot, unsigned KVH, unsigned dh, unsigned ctx, int pos) {
    if (!ensure_init(-1)) return;
    State& s = state();
    if (vsrc_off % 4) { latch("tok_v_cache: byte offset must be a multiple of 4"); return; }
    if (pos < 0 || (unsigned)pos >= ctx) { latch("tok_v_cache: position %d outside the %u-row cache", pos, ctx); return; }
    const uint8_t* v = slot_ptr(vsrcslot, vsrc_off + (size_t)KVH * dh * 4, "tok_v_cache");
    uint8_t* c = slot_ptr(cacheslot, kv_elem() * KVH * ctx * dh, "tok_v_cache");
    if (!v || !c) return;
    if (!launch_v_cache((const float*)(v + vsrc_off), c, s.kv_half, KVH, dh, ctx, pos, s.stream)) s.sticky = true;
}
void tm_cuda_tok_attn(int qslot, int kcslot, int vcslot, int probslot, int outslot, unsigned QD, unsigned H,
                      unsigned KVH, unsigned dh, unsigned ctx, int allow, float scale, unsigned REP) {
    if (!ensure_init(-1)) return;
    State& s = state();
    // the reference's argument check, metal.h:4157-4160
    if (!H || !KVH || !dh || !ctx || allow <= 0 || (unsigned)allow > ctx || H % KVH || REP != H / KVH ||
        (uint64_t)H * dh != QD || !std::isfinite(scale) || scale <= 0) {
        latch("tok_attn: invalid decode attention dimensions or scale");
        return;
    }
    const float* q = (const float*)slot_ptr(qslot, (size_t)QD * 4, "tok_attn");
    const uint8_t* kc = slot_ptr(kcslot, kv_elem() * KVH * ctx * dh, "tok_attn");
    const uint8_t* vc = slot_ptr(vcslot, kv_elem() * KVH * ctx * dh, "tok_attn");
    float* out = (float*)slot_ptr(outslot, (size_t)QD * 4, "tok_attn");
    // Split-K partials live in the probs slot, which the caller reserved for H*ctx floats.
    float* probs = (float*)slot_ptr(probslot, (size_t)H * (dh + 2) * 4, "tok_attn");
    if (!q || !kc || !vc || !out || !probs) return;
    const AttnPlan pl = plan_attention(H, KVH, dh, ctx, (unsigned)allow, s.slots[probslot].bytes);
    if (!pl.nsplit) { latch("tok_attn: probs slot too small for one split"); return; }
    if (!launch_attention(q, kc, vc, s.kv_half, probs, out, H, KVH, dh, ctx, (unsigned)allow, scale, REP, pl, s.stream)) s.sticky = true;
}
void tm_cuda_tok_argmax(int xslot, int tokslot, unsigned idx, unsigned n) {
    if (!ensure_init(-1)) return;
    State& s = state();
    const float* x = (const float*)slot_ptr(xslot, (size_t)n * 4, "tok_argmax");
    unsigned* t = (unsigned*)slot_ptr(tokslot, sizeof(unsigned) * ((size_t)idx + 1), "tok_argmax");
    unsigned long long* sc = choose_scratch();
    if (!x || !t || !sc) return;
    if (!launch_choose(x, t, n, idx, 0.f, 0u, false, sc, s.stream)) s.sticky = true;
}
void tm_cuda_tok_sample(int xslot, int tokslot, unsigned idx, unsigned n, float inv_temp, unsigned seed) {
    if (!ensure_init(-1)) return;
    State& s = state();
    const float* x = (const float*)slot_ptr(xslot, (size_t)n * 4, "tok_sample");
    unsigned* t = (unsigned*)slot_ptr(tokslot, sizeof(unsigned) * ((size_t)idx + 1), "tok_sample");
    unsigned long long* sc = choose_scratch();
    if (!x || !t || !sc) return;
    if (!launch_choose(x, t, n, idx, inv_temp, seed, true, sc, s.stream)) s.sticky = true;
}
// Reads one token without waiting for the lane: a 4-byte copy on a second stream
// (the reference polls shared memory with an acquire load, metal.h:3216-3226).
unsigned tm_cuda_tok_peek(int tokslot, unsigned idx) {
    if (!ensure_init(-1)) return 0xFFFFFFFFu;
    State& s = state();
    static cudaStream_t side = nullptr;
    if (!side && cudaStreamCreateWithFlags(&side, cudaStreamNonBlocking) != cudaSuccess) { check_launch("tok_peek"); return 0xFFFFFFFFu; }
    if (!s.peek_host && cudaMallocHost(&s.peek_host, 64) != cudaSuccess) { check_launch("tok_peek"); return 0xFFFFFFFFu; }
    if (tokslot < 0 || tokslot >= (int)s.slots.size() || !s.slots[tokslot].ptr ||
        s.slots[tokslot].bytes < sizeof(unsigned) * ((size_t)idx + 1)) { fail("tok_peek: token slot %d too small", tokslot); return 0xFFFFFFFFu; }
    if (cudaMemcpyAsync(s.peek_host, s.slots[tokslot].ptr + sizeof(unsigned) * (size_t)idx, 4, cudaMemcpyDeviceToHost, side) != cudaSuccess ||
        cudaStreamSynchronize(side) != cudaSuccess) { check_launch("tok_peek"); return 0xFFFFFFFFu; }
    return *s.peek_host;
}
void* tm_cuda_tok_slot_ptr(int slot) {
    State& s = state();
    return (slot >= 0 && slot < (int)s.slots.size()) ? s.slots[slot].ptr : nullptr;
}
void* tm_cuda_tok_stream(void) { return ensure_init(-1) ? (void*)state().stream : nullptr; }

// glue on device pointers
bool tm_cuda_rmsnorm_dev(const float* x, const float* w, float* out, unsigned D, float eps, void* stream) {
    return ensure_init(-1) && launch_rmsnorm(x, w, out, D, eps, (cudaStream_t)stream);
}
bool tm_cuda_add_dev(float* a, const float* b, unsigned n, void* stream) { return ensure_init(-1) && launch_add(a, b, n, (cudaStream_t)stream); }
bool tm_cuda_silu_mul_dev(float* g, const float* u, unsigned n, void* stream) { return ensure_init(-1) && launch_silu_mul(g, u, n, (cudaStream_t)stream); }
bool tm_cuda_argmax_dev(const float* x, unsigned* out, unsigned n, void* stream) {
    if (!ensure_init(-1)) return false;
    unsigned long long* sc = choose_scratch();
    if (!sc) return fail("argmax: scratch allocation failed");
    return launch_choose(x, out, n, 0, 0.f, 0u, false, sc, (cudaStream_t)stream);
}

// ---- chain forms: position and token index live on the device -------------------------
// A chain state is two ints in a slot: {position, token index}. The entries below read it on the
// device, so one captured CUDA graph serves every token of a greedy chain.
static const int* state_ptr(int stateslot, const char* who) { return (const int*)slot_ptr(stateslot, 16, who); }

// Exchange description of one launch. wait_site / push_site < 0: that half is absent. The flags of a
// site live at the start of the arena; y must be a shared slot when pushing (its offset in the arena
// is the same on every rank).
static bool make_exchange(Exchange& xc, int wait_site, int push_site, int stateslot, const uint8_t* y_base, const char* who) {
    State& s = state();
    PeerState& ps = s.peer;
    xc = Exchange{};
    if (wait_site < 0 && push_site < 0) return true;
    if (!ps.open) { latch("%s: the peer arena is not open", who); return false; }
    if (wait_site >= kMaxSites || push_site >= kMaxSites) { latch("%s: exchange site out of range", who); return false; }
    const int* st = (const int*)slot_ptr(stateslot, 16, who);
    if (!st) return false;
    xc.epoch = st + 3;
    xc.limit_ns = s.wait_limit_ns;
    xc.abort_local = (int*)ps.arena + kAbortWord;
    for (int q = 0; q < ps.world; ++q)
        if (q != ps.rank) xc.abort_peer[xc.npeers++] = (int*)ps.base[q] + kAbortWord;
    unsigned* ctrs = (unsigned*)ps.arena;
    if (wait_site >= 0) {
        if (!ps.site_ctas[wait_site]) { latch("%s: waits on site %d before any launch pushes to it", who, wait_site); return false; }
        xc.wait_ctrs = ctrs + (size_t)wait_site * kMaxRanks; xc.nwait = (uint32_t)ps.world; xc.self = (uint32_t)ps.rank;
        xc.wait_ctas = ps.site_ctas[wait_site];
    }
    if (push_site >= 0) {
        if (!y_base || y_base < ps.arena + kFlagBytes || y_base >= ps.arena + ps.used) { latch("%s: the pushed output must be a shared slot", who); return false; }
        const size_t off = (size_t)(y_base - ps.arena);
        uint32_t n = 0;
        for (int q = 0; q < ps.world; ++q) {
            if (q == ps.rank) continue;
            xc.peer_y[n] = (float*)(ps.base[q] + off);
            xc.peer_ctr[n] = (unsigned*)ps.base[q] + (size_t)push_site * kMaxRanks + ps.rank;
            ++n;
        }
        xc.npush = n;
    }
    return true;
}

// RMSNorm weights are cached on the device by host pointer (as tok_rmsnorm does).
static const float* norm_weights_dev(const void* norm_w, unsigned K, const char* who) {
    State& s = state();
    auto it = s.norm_w.find(norm_w);
    if (it == s.norm_w.end()) {
        float* dw = nullptr;
        if (cudaMalloc(&dw, (size_t)K * 4) != cudaSuccess) { cudaGetLastError(); latch("%s: weight allocation failed", who); return nullptr; }
        cudaMemcpyAsync(dw, norm_w, (size_t)K * 4, cudaMemcpyHostToDevice, s.stream);
        it = s.norm_w.emplace(norm_w, dw).first;
    }
    return it->second;
}

// x image (state.h): a fixed buffer, created on first use.
constexpr size_t kXImageBytes = 256 * 1024;
static bool x_images_ready() {
    State& s = state();
    static const bool on = !(std::getenv("TM_GEMV_XQ") && *std::getenv("TM_GEMV_XQ") == '0');   // A/B knob: 0 = every CTA stages x itself
    if (!on) return false;
    if (s.x_prep.buf) return true;
    uint8_t* p = nullptr;
    if (cudaMalloc(&p, kXImageBytes) != cudaSuccess) { cudaGetLastError(); return false; }
    cudaMemsetAsync(p, 0, kXImageBytes, s.stream);
    s.x_prep.buf = (uint32_t*)p;
    return true;
}
static bool image_holds(const State::XImage& im, const float* x, unsigned x_op, const float* x2, float eps, unsigned K, unsigned dtype) {
    return im.buf && im.stamp == state().launches && im.x == x && im.x_op == x_op && im.K == K && im.dtype == dtype &&
           (x_op == 0 || im.x2 == x2) && (x_op != 1 || im.eps == eps);
}

static void gemv_fused_impl(const char* who, int xslot, size_t xoff, int x_op, int x2slot, size_t x2off, const void* norm_w, float eps,
                            int wid, int yslot, size_t yoff, const size_t* seg_yoff, unsigned N, unsigned K, unsigned dtype,
                            const uint64_t* seg_woff, const unsigned* seg_rows, unsigned nseg, int accumulate,
                            int wait_site, int push_site, int stateslot) {
    if (!ensure_init(-1)) return;
    State& s = state();
    const size_t row_bytes = weight_bytes(dtype, 1, K);
    if (!row_bytes) { latch("%s: K=%u is not whole blocks of dtype %u", who, K, dtype); return; }
    if (yoff % 4 || xoff % 16 || x2off % 16) { latch("%s: misaligned byte offset", who); return; }
    SegTable t;
    if (!make_segments(t, N, seg_woff, seg_rows, nseg)) { s.sticky = true; return; }
    const int i = wid - kFirstWeight;
    if (i < 0 || i >= (int)s.wbufs.size() || !s.wbufs[i].ptr) { latch("%s: unknown weight handle %d", who, wid); return; }
    for (unsigned k = 0; k < nseg; ++k)
        if (t.woff[k] > s.wbufs[i].bytes || (size_t)seg_rows[k] * row_bytes > s.wbufs[i].bytes - t.woff[k]) {
            latch("%s: segment %u lies outside weight handle %d", who, k, wid); return;
        }
    size_t y_need = yoff + (size_t)N * 4;
    if (seg_yoff) {                                          // every segment lands at its own byte offset of the slot
        y_need = 0;
        for (unsigned k = 0; k < nseg; ++k) {
            if (seg_yoff[k] % 4) { latch("%s: misaligned output offset", who); return; }
            t.yoff[k] = (uint32_t)(seg_yoff[k] / 4);
            const size_t end = seg_yoff[k] + (size_t)seg_rows[k] * 4;
            y_need = end > y_need ? end : y_need;
        }
        yoff = 0;
    }
    const uint8_t* x = slot_ptr(xslot, xoff + (size_t)K * 4, who);
    uint8_t* y = slot_ptr(yslot, y_need, who);
    if (!x || !y) return;
    Exchange xc;
    if (!make_exchange(xc, wait_site, push_site, stateslot, y + yoff, who)) return;
    GemvFuse f{};
    f.x_op = (unsigned)x_op; f.eps = eps; f.accumulate = accumulate != 0; f.x2 = nullptr;
    f.xchg = (xc.nwait || xc.npush) ? &xc : nullptr;
    if (x_op == 1) {
        if (!norm_w) { latch("%s: rmsnorm needs its weights", who); return; }
        f.x2 = norm_weights_dev(norm_w, K, who);
        if (!f.x2) return;
    } else if (x_op == 2) {
        const uint8_t* u = slot_ptr(x2slot, x2off + (size_t)K * 4, who);
        if (!u) return;
        f.x2 = (const float*)(u + x2off);
    } else if (x_op != 0) { latch("%s: unknown x transform %d", who, x_op); return; }
    // Heavy staging (SiLU * up, or a long K) is done once per launch by a small kernel ahead of the GEMV instead of by
    // every CTA; a GEMV that follows on the same x (k and v after q) reuses the image. Light staging stays in the CTAs:
    // there the extra dependent kernel costs what it saves.
    const float* xp = (const float*)(x + xoff);
    float* yp = (float*)(y + yoff);
    State::XImage* used = nullptr;
    const size_t img = xq_bytes(K, dtype);
    if ((f.x_op == 2 || K >= 8192) && img && img <= kXImageBytes && x_images_ready()) {
        if (!(wait_site < 0 && image_holds(s.x_prep, xp, f.x_op, f.x2, eps, K, dtype))) {
            Exchange xw = xc;
            xw.npush = 0;                                    // the staging kernel only waits for the gather, it pushes nothing
            if (!launch_xprep(s.x_prep.buf, xp, f.x2, f.x_op, eps, K, dtype, xw.nwait ? &xw : nullptr, s.stream)) { s.sticky = true; return; }
            s.x_prep.x = xp; s.x_prep.x2 = f.x2; s.x_prep.x_op = f.x_op; s.x_prep.K = K; s.x_prep.dtype = dtype; s.x_prep.eps = eps;
        }
        used = &s.x_prep;
        f.xq = used->buf;
    }
    if (!launch_gemv(xp, s.wbufs[i].ptr, yp, N, K, dtype, t, s.stream, &f)) { s.sticky = true; return; }
    // The image stays current while the launches that follow its producer only read it: this GEMV did, unless its output
    // overlaps the x the image was made from.
    if (used) {
        const bool clobbers = (const uint8_t*)yp < (const uint8_t*)xp + (size_t)K * 4 && (const uint8_t*)xp < y + y_need;
        used->stamp = clobbers ? ~0ull : s.launches;
    }
    if (push_site >= 0) {
        // every rank launches the same shapes, so this grid is also what the peers' counters advance by per token
        unsigned& ctas = s.peer.site_ctas[push_site];
        if (ctas && ctas != last_gemv_grid()) latch("%s: site %d was pushed to by %u CTAs before, now by %u", who, push_site, ctas, last_gemv_grid());
        ctas = last_gemv_grid();
    }
}

void tm_cuda_tok_gemv_fused(int xslot, size_t xoff, int x_op, int x2slot, size_t x2off, const void* norm_w, float eps,
                            int wid, int yslot, size_t yoff, unsigned N, unsigned K, unsigned dtype,
                            const uint64_t* seg_woff, const unsigned* seg_rows, unsigned nseg, int accumulate) {
    gemv_fused_impl("tok_gemv_fused", xslot, xoff, x_op, x2slot, x2off, norm_w, eps, wid, yslot, yoff, nullptr, N, K, dtype,
                    seg_woff, seg_rows, nseg, accumulate, -1, -1, -1);
}
void tm_cuda_tok_gemv_xchg(int xslot, size_t xoff, int x_op, int x2slot, size_t x2off, const void* norm_w, float eps,
                           int wid, int yslot, const size_t* seg_yoff, unsigned N, unsigned K, unsigned dtype,
                           const uint64_t* seg_woff, const unsigned* seg_rows, unsigned nseg, int accumulate,
                           int wait_site, int push_site, int stateslot) {
    if (!seg_yoff) { if (ensure_init(-1)) latch("tok_gemv_xchg: null output offsets"); return; }
    gemv_fused_impl("tok_gemv_xchg", xslot, xoff, x_op, x2slot, x2off, norm_w, eps, wid, yslot, 0, seg_yoff, N, K, dtype,
                    seg_woff, seg_rows, nseg, accumulate, wait_site, push_site, stateslot);
}
void tm_cuda_tok_qkv_post_at(int qkvslot, int kcslot, int vcslot, unsigned H, unsigned KVH, unsigned dh, unsigned ctx,
                             float theta, int stateslot) {
    if (!ensure_init(-1)) return;
    State& s = state();
    if (!ensure_rope(dh, ctx, theta)) return;
    float* qkv = (float*)slot_ptr(qkvslot, (size_t)(H + 2 * KVH) * dh * 4, "tok_qkv_post_at");
    uint8_t* kc = slot_ptr(kcslot, kv_elem() * KVH * ctx * dh, "tok_qkv_post_at");
    uint8_t* vc = slot_ptr(vcslot, kv_elem() * KVH * ctx * dh, "tok_qkv_post_at");
    const int* st = state_ptr(stateslot, "tok_qkv_post_at");
    if (!qkv || !kc || !vc || !st) return;
    if (!launch_qkv_post(qkv, kc, vc, s.kv_half, H, KVH, dh, ctx, s.rope_tbl, s.rope_cap * (dh / 2), st, s.stream)) s.sticky = true;
}
void tm_cuda_tok_attn_at(int qslot, int kcslot, int vcslot, int probslot, int outslot, unsigned QD, unsigned H,
                         unsigned KVH, unsigned dh, unsigned ctx, float scale, unsigned REP, int stateslot) {
    if (!ensure_init(-1)) return;
    State& s = state();
    if (!H || !KVH || !dh || !ctx || H % KVH || REP != H / KVH || (uint64_t)H * dh != QD || !std::isfinite(scale) || scale <= 0) {
        latch("tok_attn_at: invalid decode attention dimensions or scale");
        return;
    }
    const float* q = (const float*)slot_ptr(qslot, (size_t)QD * 4, "tok_attn_at");
    const uint8_t* kc = slot_ptr(kcslot, kv_elem() * KVH * ctx * dh, "tok_attn_at");
    const uint8_t* vc = slot_ptr(vcslot, kv_elem() * KVH * ctx * dh, "tok_attn_at");
    float* out = (float*)slot_ptr(outslot, (size_t)QD * 4, "tok_attn_at");
    float* probs = (float*)slot_ptr(probslot, (size_t)H * (dh + 2) * 4, "tok_attn_at");
    const int* st = state_ptr(stateslot, "tok_attn_at");
    if (!q || !kc || !vc || !out || !probs || !st) return;
    // the split count is fixed for the whole chain (sized for a full context); the kernel derives its chunk from the state
    const AttnPlan pl = plan_attention(H, KVH, dh, ctx, ctx, s.slots[probslot].bytes);
    if (!pl.nsplit) { latch("tok_attn_at: probs slot too small for one split"); return; }
    if (!launch_attention(q, kc, vc, s.kv_half, probs, out, H, KVH, dh, ctx, ctx, scale, REP, pl, s.stream, st)) s.sticky = true;
}
void tm_cuda_tok_attn_fused_at(int qkvslot, int kcslot, int vcslot, int probslot, int outslot, unsigned H, unsigned KVH,
                               unsigned dh, unsigned ctx, float scale, float theta, int stateslot) {
    if (!ensure_init(-1)) return;
    State& s = state();
    const char* who = "tok_attn_fused_at";
    if (!H || !KVH || !dh || !ctx || H % KVH || !std::isfinite(scale) || scale <= 0) { latch("%s: invalid attention dimensions or scale", who); return; }
    if (!ensure_rope(dh, ctx, theta)) return;
    const float* qkv = (const float*)slot_ptr(qkvslot, (size_t)(H + 2 * KVH) * dh * 4, who);
    uint8_t* kc = slot_ptr(kcslot, kv_elem() * KVH * ctx * dh, who);
    uint8_t* vc = slot_ptr(vcslot, kv_elem() * KVH * ctx * dh, who);
    float* out = (float*)slot_ptr(outslot, (size_t)H * dh * 4, who);
    float* probs = (float*)slot_ptr(probslot, (size_t)H * (dh + 2) * 4, who);
    const int* st = state_ptr(stateslot, who);
    if (!qkv || !kc || !vc || !out || !probs || !st) return;
    if (!launch_attn_fused(qkv, kc, vc, s.kv_half, probs, s.slots[probslot].bytes, out, H, KVH, dh, ctx, scale, s.rope_tbl,
                           s.rope_cap * (dh / 2), st, s.stream)) s.sticky = true;
}
static void argmax_at_impl(const char* who, int xslot, int tokslot, unsigned n, unsigned max_tokens, int stateslot, int wait_site,
                           bool sample = false, float inv_temp = 0.f, unsigned seed = 0u) {
    if (!ensure_init(-1)) return;
    State& s = state();
    const float* x = (const float*)slot_ptr(xslot, (size_t)n * 4, who);
    unsigned* t = (unsigned*)slot_ptr(tokslot, sizeof(unsigned) * (size_t)max_tokens, who);
    const int* st = state_ptr(stateslot, who);
    unsigned long long* sc = choose_scratch();
    if (!x || !t || !st || !sc) return;
    Exchange xc;
    if (!make_exchange(xc, wait_site, -1, stateslot, nullptr, who)) return;
    if (!launch_choose(x, t, n, 0, inv_temp, seed, sample, sc, s.stream, st, xc.nwait ? &xc : nullptr)) s.sticky = true;
}
void tm_cuda_tok_sample_at(int xslot, int tokslot, unsigned n, unsigned max_tokens, float inv_temp, unsigned seed, int stateslot,
                           int wait_site) {
    argmax_at_impl("tok_sample_at", xslot, tokslot, n, max_tokens, stateslot, wait_site, true, inv_temp, seed);
}
void tm_cuda_tok_argmax_at(int xslot, int tokslot, unsigned n, unsigned max_tokens, int stateslot) {
    argmax_at_impl("tok_argmax_at", xslot, tokslot, n, max_tokens, stateslot, -1);
}
void tm_cuda_tok_argmax_xchg(int xslot, int tokslot, unsigned n, unsigned max_tokens, int stateslot, int wait_site) {
    argmax_at_impl("tok_argmax_xchg", xslot, tokslot, n, max_tokens, stateslot, wait_site);
}
void tm_cuda_tok_choose_shard(int xslot, unsigned lo, unsigned n_local, unsigned n_total, int tokslot, unsigned max_tokens,
                              float inv_temp, unsigned seed, int stateslot, int keyslot, int site) {
    const char* who = "tok_choose_shard";
    if (!ensure_init(-1)) return;
    State& s = state();
    PeerState& ps = s.peer;
    if (!ps.open) { latch("%s: the peer arena is not open", who); return; }
    if (site < 0 || site >= kMaxSites) { latch("%s: exchange site out of range", who); return; }
    if (n_local == 0 || (uint64_t)lo + n_local > n_total) { latch("%s: rows [%u, %u) are not inside %u", who, lo, lo + n_local, n_total); return; }
    const float* x = (const float*)slot_ptr(xslot, (size_t)n_total * 4, who);
    unsigned* t = (unsigned*)slot_ptr(tokslot, sizeof(unsigned) * (size_t)max_tokens, who);
    const int* st = state_ptr(stateslot, who);
    unsigned long long* keys = (unsigned long long*)slot_ptr(keyslot, sizeof(unsigned long long) * (size_t)ps.world, who);
    unsigned long long* sc = choose_scratch();
    if (!x || !t || !st || !keys || !sc) return;
    if ((uintptr_t)keys % 8) { latch("%s: the key table must be 8-byte aligned", who); return; }
    unsigned& ctas = ps.site_ctas[site];
    if (ctas && ctas != 1) { latch("%s: site %d was pushed to by %u CTAs before; a key exchange counts once per rank", who, site, ctas); return; }
    ctas = 1;
    Exchange xc;
    if (!make_exchange(xc, site, site, stateslot, (const uint8_t*)keys, who)) return;
    if (!launch_choose_shard(x, t, lo, n_local, inv_temp, seed, inv_temp > 0.f, sc, keys, s.stream, st, xc)) s.sticky = true;
}
void tm_cuda_tok_embed_at(int tokslot, int wid, uint64_t woff, int xslot, unsigned D, unsigned dtype, unsigned max_tokens,
                          int stateslot) {
    if (!ensure_init(-1)) return;
    State& s = state();
    const unsigned* tok = (const unsigned*)slot_ptr(tokslot, sizeof(unsigned) * (size_t)max_tokens, "tok_embed_at");
    float* x = (float*)slot_ptr(xslot, (size_t)D * 4, "tok_embed_at");
    const uint8_t* W = weight_ptr(wid, woff, 0, "tok_embed_at");
    const int* st = state_ptr(stateslot, "tok_embed_at");
    if (!tok || !x || !W || !st) return;
    if (!launch_embed_row(tok, 0, W, x, D, dtype, s.stream, st)) s.sticky = true;
}
void tm_cuda_tok_advance(int stateslot) {
    if (!ensure_init(-1)) return;
    int* st = (int*)slot_ptr(stateslot, 16, "tok_advance");
    if (st && !launch_advance(st, state().stream)) state().sticky = true;
}

// ---- CUDA graphs over the lane -----------------------------------------------------------
// Everything encoded between graph_begin and graph_end is captured instead of executed; the
// resulting graph replays the same launches (same slots, same weight handles). Slots, weight
// handles, norm weights and the rope table must exist before the capture starts: run the
// sequence once eagerly first.
static std::vector<cudaGraphExec_t>& graphs() { static std::vector<cudaGraphExec_t> g; return g; }
bool tm_cuda_tok_graph_begin(void) {
    if (!ensure_init(-1)) return false;
    State& s = state();
    if (s.capturing) return fail("tok_graph_begin: a capture is already open");
    if (cudaStreamBeginCapture(s.stream, cudaStreamCaptureModeRelaxed) != cudaSuccess) return check_launch("tok_graph_begin");
    s.capturing = true; s.encoding = true; s.sticky = false;
    return true;
}
int tm_cuda_tok_graph_end(void) {
    State& s = state();
    if (!s.ready || !s.capturing) { fail("tok_graph_end: no capture is open"); return -1; }
    cudaGraph_t g = nullptr;
    const cudaError_t e = cudaStreamEndCapture(s.stream, &g);
    s.capturing = false; s.encoding = false;
    const bool sticky = s.sticky; s.sticky = false;
    if (e != cudaSuccess || !g) { cudaGetLastError(); fail("tok_graph_end: %s", cudaGetErrorString(e)); return -1; }
    if (sticky) { cudaGraphDestroy(g); ++s.fallbacks; return -1; }
    cudaGraphExec_t x = nullptr;
    if (cudaGraphInstantiate(&x, g, 0) != cudaSuccess) { cudaGraphDestroy(g); check_launch("tok_graph_end: instantiate"); return -1; }
    cudaGraphDestroy(g);
    graphs().push_back(x);
    return (int)graphs().size() - 1;
}
bool tm_cuda_tok_graph_launch(int id, unsigned times) {
    if (!ensure_init(-1)) return false;
    State& s = state();
    if (id < 0 || id >= (int)graphs().size() || !graphs()[id]) return fail("tok_graph_launch: unknown graph %d", id);
    for (unsigned i = 0; i < times; ++i)
        if (cudaGraphLaunch(graphs()[id], s.stream) != cudaSuccess) return check_launch("tok_graph_launch");
    return true;
}
void tm_cuda_tok_graph_destroy(int id) {
    if (id < 0) {                                            // every graph of the lane
        for (cudaGraphExec_t& g : graphs()) if (g) { cudaGraphExecDestroy(g); g = nullptr; }
        return;
    }
    if (id >= 0 && id < (int)graphs().size() && graphs()[id]) { cudaGraphExecDestroy(graphs()[id]); graphs()[id] = nullptr; }
}

size_t tm_cuda_attn_decode_scratch(unsigned H, unsigned KVH, unsigned dh, unsigned ctx, unsigned allow) {
    if (!ensure_init(-1) || !H || !KVH || !dh || !allow) return 0;
    const AttnPlan pl = plan_attention(H, KVH, dh, ctx, allow, (size_t)1 << 40);
    return (size_t)pl.nsplit * H * (dh + 2) * sizeof(float);
}
bool tm_cuda_attn_decode_dev(const float* q, const void* kc, const void* vc, float* scratch, size_t scratch_bytes,
                             float* out, unsigned H, unsigned KVH, unsigned dh, unsigned ctx, unsigned allow,
                             float scale, int kv_half, void* stream) {
    if (!ensure_init(-1)) return false;
    if (!q || !kc || !vc || !scratch || !out) return fail("attn_decode: null pointer");
    if (!H || !KVH || !dh || !ctx || !allow || allow > ctx || H % KVH || !std::isfinite(scale) || scale <= 0)
        return fail("attn_decode: invalid decode attention dimensions or scale");
    const AttnPlan pl = plan_attention(H, KVH, dh, ctx, allow, scratch_bytes);
    if (!pl.nsplit) return fail("attn_decode: scratch of %zu bytes cannot hold one split", scratch_bytes);
    return launch_attention(q, kc, vc, kv_half != 0, scratch, out, H, KVH, dh, ctx, allow, scale, H / KVH, pl,
                            (cudaStream_t)stream);
}

// ---- the reference's symbol names (tensormark/metal_shim.mm:22-152) -------------------
bool tm_metal_tok_begin(void) { return tm_cuda_tok_begin(); }
bool tm_metal_tok_flush(void) { return tm_cuda_tok_flush(); }
bool tm_metal_tok_end(int o, float* d, unsigned n) { return tm_cuda_tok_end(o, d, n); }
bool tm_metal_tok_end_async(void) { return tm_cuda_tok_end_async(); }
bool tm_metal_tok_wait_pending(void) { return tm_cuda_tok_wait_pending(); }
bool tm_metal_tok_reserve(int s, size_t b) { return tm_cuda_tok_reserve(s, b); }
bool tm_metal_tok_upload(int s, size_t o, const void* p, size_t b) { return tm_cuda_tok_upload(s, o, p, b); }
bool tm_metal_tok_download(int s, size_t o, void* p, size_t b) { return tm_cuda_tok_download(s, o, p, b); }
bool tm_metal_tok_kv_reserve(int s, size_t n) { return tm_cuda_tok_kv_reserve(s, n); }
bool tm_metal_tok_kv_upload(int s, size_t o, const float* p, size_t n) { return tm_cuda_tok_kv_upload(s, o, p, n); }
bool tm_metal_tok_kv_download(int s, size_t o, float* p, size_t n) { return tm_cuda_tok_kv_download(s, o, p, n); }
int tm_metal_tok_wbuf(const void* t, size_t b, const void* mb, size_t ms, int z, uint64_t* w) { return tm_cuda_tok_wbuf(t, b, mb, ms, z, w); }
bool tm_metal_tok_probe_copy(int a, size_t o, int d, unsigned n) { return tm_cuda_tok_probe_copy(a, o, d, n); }
void tm_metal_tok_gemv(int x, int w, uint64_t wo, int y, size_t yo, unsigned N, unsigned K) { tm_cuda_tok_gemv(x, w, wo, y, yo, N, K); }
bool tm_metal_tok_gemv_seg_supported(unsigned dt) { return tm_cuda_tok_gemv_seg_supported(dt); }
void tm_metal_tok_gemv_seg(int x, int w, int y, size_t yo, unsigned N, unsigned K, const uint64_t* so, const unsigned* sr, unsigned ns) { tm_cuda_tok_gemv_seg(x, w, y, yo, N, K, so, sr, ns); }
void tm_metal_tok_gemv_seg_dt(int x, int w, int y, size_t yo, unsigned N, unsigned K, unsigned dt, const uint64_t* so, const unsigned* sr, unsigned ns) { tm_cuda_tok_gemv_seg_dt(x, w, y, yo, N, K, dt, so, sr, ns); }
void tm_metal_tok_gemv_kq(int x, int w, uint64_t wo, int y, size_t yo, unsigned N, unsigned K, unsigned dt) { tm_cuda_tok_gemv_kq(x, w, wo, y, yo, N, K, dt); }
void tm_metal_tok_embed_q4(int t, unsigned i, int w, uint64_t wo, int x, unsigned D) { tm_cuda_tok_embed_q4(t, i, w, wo, x, D); }
void tm_metal_tok_embed_kq(int t, unsigned i, int w, uint64_t wo, int x, unsigned D, unsigned dt) { tm_cuda_tok_embed_kq(t, i, w, wo, x, D, dt); }
void tm_metal_tok_gemv_h(int x, int w, uint64_t wo, int y, size_t yo, unsigned N, unsigned K) { tm_cuda_tok_gemv_h(x, w, wo, y, yo, N, K); }
void tm_metal_tok_embed_h(int t, unsigned i, int w, uint64_t wo, int x, unsigned D) { tm_cuda_tok_embed_h(t, i, w, wo, x, D); }
void tm_metal_tok_bias_qkv(int y, int b, size_t bo, unsigned N) { tm_cuda_tok_bias_qkv(y, b, bo, N); }
void tm_metal_tok_rmsnorm(int x, const void* w, int o, unsigned D, float eps) { tm_cuda_tok_rmsnorm(x, w, o, D, eps); }
void tm_metal_tok_add(int a, int b, unsigned n) { tm_cuda_tok_add(a, b, n); }
void tm_metal_tok_silu_mul(int g, size_t go, int u, size_t uo, unsigned n) { tm_cuda_tok_silu_mul(g, go, u, uo, n); }
void tm_metal_tok_rope_q(int q, unsigned H, unsigned dh, int pos, float th) { tm_cuda_tok_rope_q(q, H, dh, pos, th); }
void tm_metal_tok_rope_k_cache(int k, size_t ko, int c, unsigned KVH, unsigned dh, unsigned ctx, int pos, float th) { tm_cuda_tok_rope_k_cache(k, ko, c, KVH, dh, ctx, pos, th); }
void tm_metal_tok_v_cache(int v, size_t vo, int c, unsigned KVH, unsigned dh, unsigned ctx, int pos) { tm_cuda_tok_v_cache(v, vo, c, KVH, dh, ctx, pos); }
void tm_metal_tok_attn(int q, int kc, int vc, int pr, int o, unsigned QD, unsigned H, unsigned KVH, unsigned dh, unsigned ctx, int allow, float sc, unsigned REP) { tm_cuda_tok_attn(q, kc, vc, pr, o, QD, H, KVH, dh, ctx, allow, sc, REP); }
void tm_metal_tok_argmax(int x, int t, unsigned i, unsigned n) { tm_cuda_tok_argmax(x, t, i, n); }
void tm_metal_tok_sample(int x, int t, unsigned i, unsigned n, float it, unsigned sd) { tm_cuda_tok_sample(x, t, i, n, it, sd); }
unsigned tm_metal_tok_peek(int t, unsigned i) { return tm_cuda_tok_peek(t, i); }

}  // extern "C"
