// peer.cu — peer-mapped arena of a row-sharded model: one process per GPU, each rank's arena mapped
// into every other rank through CUDA IPC, so kernels store straight into the peers' buffers over
// NVLink (the all-gather fused into the GEMV, struct Exchange in common.cuh).
//
// No counterpart in the reference (single GPU). Set-up, on every rank, in this order:
//   tm_cuda_init(device); tm_cuda_peer_arena(bytes, handle)      allocate and export
//   <exchange the handles between the ranks, any channel>
//   tm_cuda_peer_open(rank, world, handles)                      map the peers
//   tm_cuda_tok_reserve_shared(slot, bytes) ...                  same order on every rank
// and, before the process ends, tm_cuda_peer_unmap() on every rank, a barrier, tm_cuda_peer_close().
#include "cuda_shim.h"
#include "common.cuh"
#include "state.h"

#include <cstring>

using namespace tmc;

extern "C" {

size_t tm_cuda_peer_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

bool tm_cuda_peer_arena(size_t bytes, void* handle_out) {
    if (!ensure_init(-1)) return false;
    PeerState& ps = state().peer;
    if (ps.arena) return fail("peer: the arena already exists");
    if (!handle_out) return fail("peer: null handle buffer");
    const size_t want = (kFlagBytes + bytes + 4095) / 4096 * 4096;
    uint8_t* p = nullptr;
    if (cudaMalloc(&p, want) != cudaSuccess) { cudaGetLastError(); return fail("peer: arena allocation of %zu bytes failed", want); }
    if (cudaMemset(p, 0, want) != cudaSuccess) { cudaFree(p); return check_launch("peer: arena clear"); }
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) { cudaFree(p); return check_launch("peer: cudaIpcGetMemHandle"); }
    std::memcpy(handle_out, &h, sizeof h);
    ps.arena = p; ps.bytes = want; ps.used = kFlagBytes;
    return true;
}

bool tm_cuda_peer_open(int rank, int world, const void* handles) {
    if (!ensure_init(-1)) return false;
    PeerState& ps = state().peer;
    if (!ps.arena) return fail("peer: create the arena first");
    if (ps.open) return fail("peer: already open");
    if (world < 2 || world > kMaxRanks || rank < 0 || rank >= world || !handles) return fail("peer: rank %d of %d is not valid (2..%d ranks)", rank, world, kMaxRanks);
    for (int q = 0; q < world; ++q) {
        if (q == rank) { ps.base[q] = ps.arena; continue; }
        cudaIpcMemHandle_t h;
        std::memcpy(&h, (const uint8_t*)handles + (size_t)q * sizeof h, sizeof h);
        void* p = nullptr;
        if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            for (int k = 0; k < q; ++k) if (k != rank && ps.base[k]) { cudaIpcCloseMemHandle(ps.base[k]); ps.base[k] = nullptr; }
            return check_launch("peer: cudaIpcOpenMemHandle");
        }
        ps.base[q] = (uint8_t*)p;
    }
    ps.rank = rank; ps.world = world; ps.open = true;
    return true;
}

// Single-GPU rehearsal of the sharded lane: every "peer" arena is this GPU's own arena. Pushed rows and counts land
// in local memory; the counters of the other ranks never advance, so a kernel that waits for them runs into its
// limit, which is how the give-up path (status word, abort word) is exercised without a second GPU.
bool tm_cuda_peer_open_loopback(int rank, int world) {
    if (!ensure_init(-1)) return false;
    PeerState& ps = state().peer;
    if (!ps.arena) return fail("peer: create the arena first");
    if (ps.open) return fail("peer: already open");
    if (world < 2 || world > kMaxRanks || rank < 0 || rank >= world) return fail("peer: rank %d of %d is not valid (2..%d ranks)", rank, world, kMaxRanks);
    for (int q = 0; q < world; ++q) ps.base[q] = ps.arena;
    ps.rank = rank; ps.world = world; ps.open = true; ps.loopback = true;
    return true;
}

// Rehearsals (tests, tools): advance rank `rank`'s counter of `site` in THIS arena by `count`, in stream order, as
// that rank's pushes would; with the loopback arena this is how a test plays the part of the other ranks.
__global__ void peer_bump_kernel(unsigned* ctr, unsigned count) { atomicAdd_system(ctr, count); }
bool tm_cuda_peer_bump(int site, int rank, unsigned count) {
    if (!ensure_init(-1)) return false;
    State& s = state();
    PeerState& ps = s.peer;
    if (!ps.open) return fail("peer: the arena is not open");
    if (site < 0 || site >= kMaxSites || rank < 0 || rank >= ps.world) return fail("peer: site %d / rank %d out of range", site, rank);
    peer_bump_kernel<<<1, 1, 0, s.stream>>>((unsigned*)ps.arena + (size_t)site * kMaxRanks + rank, count);
    return check_launch("peer_bump");
}

int tm_cuda_peer_world(void) { return state().peer.open ? state().peer.world : 1; }
int tm_cuda_peer_rank(void) { return state().peer.open ? state().peer.rank : 0; }

// Two-phase teardown: every rank unmaps its peers, the ranks meet (a barrier of the caller), then every
// rank frees its own arena, so no arena is freed while a peer still has it mapped.
bool tm_cuda_peer_unmap(void) {
    State& s = state();
    PeerState& ps = s.peer;
    if (!ps.open) return true;
    if (s.ready) cudaStreamSynchronize(s.stream);
    for (int q = 0; q < ps.world; ++q) {
        if (q != ps.rank && ps.base[q] && !ps.loopback) cudaIpcCloseMemHandle(ps.base[q]);
        if (q != ps.rank) ps.base[q] = nullptr;
    }
    ps.open = false; ps.loopback = false;
    return check_launch("peer: unmap");
}

bool tm_cuda_peer_close(void) {
    State& s = state();
    PeerState& ps = s.peer;
    if (!ps.arena) return true;
    tm_cuda_peer_unmap();
    for (Slot& sl : s.slots) if (sl.shared) { sl.ptr = nullptr; sl.bytes = 0; sl.shared = false; }
    cudaFree(ps.arena);
    ps = PeerState{};
    return check_launch("peer: close");
}

bool tm_cuda_tok_reserve_shared(int slot, size_t bytes) {
    if (!ensure_init(-1)) return false;
    State& s = state();
    PeerState& ps = s.peer;
    if (!ps.arena) return fail("tok_reserve_shared: no peer arena");
    if (s.encoding) return fail("tok_reserve_shared: not while a token is encoded");
    if (slot < 0 || slot >= 1000 || bytes == 0) return fail("tok_reserve_shared: bad slot %d or size", slot);
    if ((int)s.slots.size() <= slot) s.slots.resize((size_t)slot + 1);
    Slot& sl = s.slots[slot];
    if (sl.shared) return sl.bytes >= bytes ? true : fail("tok_reserve_shared: slot %d is shared and holds %zu bytes, %zu wanted", slot, sl.bytes, bytes);
    if (sl.ptr) return fail("tok_reserve_shared: slot %d already exists as a private slot", slot);
    const size_t want = (bytes + 255) / 256 * 256;
    if (ps.used + want > ps.bytes) return fail("tok_reserve_shared: the arena is full (%zu of %zu bytes used, %zu wanted)", ps.used, ps.bytes, want);
    sl.ptr = ps.arena + ps.used; sl.bytes = want; sl.shared = true;
    ps.used += want;
    return true;
}

}  // extern "C"
