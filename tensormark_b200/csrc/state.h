// state.h — process-wide state of the CUDA backend (one device, one lane).
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <map>
#include <string>
#include <utility>
#include <vector>

#include "common.cuh"

namespace tmc {

struct Scratch {                 // grow-only device buffer
    void* ptr = nullptr;
    size_t cap = 0;
    void* get(size_t bytes);     // nullptr when the allocation fails
    void release();
};

struct Slot {                    // token-lane slot: backend-owned device buffer (tensormark/metal.h:2262-2281)
    uint8_t* ptr = nullptr;
    size_t bytes = 0;
    bool shared = false;         // carved from the peer arena: never grown, never freed on its own
};

// Row-sharded models: this rank's arena (exported to the peers) and the peers' arenas mapped here.
// The arena starts with the exchange counters, counters[site][rank]; shared slots follow, at the same
// offsets on every rank because every rank reserves them in the same order.
constexpr int kMaxRanks = 8, kMaxSites = 256;
constexpr size_t kAbortWord = (size_t)kMaxSites * kMaxRanks;      // index (in ints) of the arena's sticky abort word
constexpr size_t kFlagBytes = (kAbortWord + 64) * sizeof(int);
struct PeerState {
    uint8_t* arena = nullptr;
    size_t bytes = 0, used = 0;
    uint8_t* base[kMaxRanks] = {};                              // base[rank] == arena once opened
    int rank = 0, world = 1;
    bool open = false;
    bool loopback = false;                                      // every peer base is this GPU's own arena (single-GPU rehearsal)
    unsigned site_ctas[kMaxSites] = {};                         // CTAs of the launch that pushes to each site (0: none yet)
};

struct WeightBuf {               // registered weights: handle id = 1000 + index (metal.h:3282-3337)
    uint8_t* ptr = nullptr;
    size_t bytes = 0;
};

struct State {
    bool ready = false, verbose = false, kv_half = true;
    unsigned long long wait_limit_ns = 2000000000ull;           // bounded device waits on other GPUs (TM_CUDA_WAIT_LIMIT_MS)
    int device = -1, sm_count = 0;
    cudaStream_t stream = nullptr;
    int* status_dev = nullptr;                                  // device view of status_host
    volatile int* status_host = nullptr;                        // pinned, mapped: kernels store a code here when a bounded wait runs out
    unsigned long long* trace_dev = nullptr;                    // TM_CUDA_TRACE=1: [0] = launches recorded, then kTraceWords per launch
    std::string last_error;
    unsigned long long fallbacks = 0, launches = 0;

    // per-tensor host-pointer entries
    std::map<std::pair<const void*, size_t>, uint8_t*> wcache;
    Scratch io_x, io_y, io_big, io_a, io_xq, gemm_ws;

    // token lane
    std::vector<Slot> slots;
    std::vector<WeightBuf> wbufs;
    std::map<const void*, std::pair<int, uint64_t>> wreg;      // tensor pointer -> (handle, byte offset)
    const void* shared_base = nullptr;                          // host base of the mapping held by shared_id
    int shared_id = -1;
    std::map<const void*, float*> norm_w;                       // rmsnorm weights cached by host pointer
    bool encoding = false;                                      // between tok_begin and the matching end
    bool capturing = false;                                     // between tok_graph_begin and tok_graph_end
    bool sticky = false;                                        // a void encoder failed since the last end
    std::vector<cudaEvent_t> pending;                           // tok_end_async markers
    float* rope_tbl = nullptr;                                  // (cos, sin) pairs [cap][dh/2]
    unsigned rope_dh = 0, rope_cap = 0;
    float rope_theta = 0.f;
    unsigned* peek_host = nullptr;                              // pinned mirror for tok_peek
    PeerState peer;

    // x image of the chain forms: x in the GEMV lanes' unit form, written once per launch by the xprep kernel.
    // A fixed-size buffer, so that captured graphs keep a valid pointer.
    struct XImage {
        uint32_t* buf = nullptr;
        const float* x = nullptr; const float* x2 = nullptr;    // what the image holds: x after (x_op, x2, eps), for (K, dtype)
        unsigned x_op = 0, K = 0, dtype = 0;
        float eps = 0.f;
        unsigned long long stamp = ~0ull;                       // value of `launches` up to which the image is known to be current
    };
    XImage x_prep;
};

State& state();
bool ensure_init(int device);
bool harvest_status(const char* where);
bool sync_stream(cudaStream_t st, const char* where);
const uint8_t* cached_weights(const void* host, size_t bytes);
// token_lane.cu, for the prefill layer stack: device address of a registered weight range (nullptr + latched error when
// outside the handle), the shared (cos, sin) rope table grown to `need` positions, a slot's device address.
const uint8_t* lane_weight_ptr(int wid, uint64_t woff, size_t bytes);
const float* lane_rope_table(unsigned dh, unsigned need, float theta, unsigned* entries);
uint8_t* lane_slot_ptr(int sid, size_t bytes, const char* who);
SegTable one_segment(unsigned N);
bool make_segments(SegTable& t, unsigned N, const uint64_t* seg_woff, const unsigned* seg_rows, unsigned nseg);

}  // namespace tmc
