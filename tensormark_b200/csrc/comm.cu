// comm.cu — the lane's one collective: an fp32 all-gather between the ranks of a row-sharded model.
//
// The reference runs on a single GPU and has no counterpart for this file. A model whose FFN and
// LM-head rows are spread over several GPUs (one process per GPU) needs every rank to see the whole
// output vector after each sharded GEMV; the lane gets that from ncclAllGather, enqueued on the lane's
// stream like any other op, so it is captured into the per-token CUDA graph with the kernels around it.
//
// NCCL is bound at run time (dlopen of libnccl.so.2, the library a torch process already holds), so a
// single-GPU user of libtm_cuda.so needs no NCCL at all. Only five functions are used; their
// prototypes below follow NCCL's public header. The unique id is produced by rank 0 and carried to
// the other ranks by the caller (torch.distributed, MPI, a file: any channel for 128 bytes).
//
// Teardown order matters: graphs that captured a collective hold the communicator, so every graph
// of the lane is destroyed before the communicator is.
#include "cuda_shim.h"
#include "common.cuh"
#include "state.h"

#include <dlfcn.h>

#include <cstring>

namespace tmc {
namespace {

struct NcclComm;
struct NcclUniqueId { char internal[128]; };
constexpr int kNcclFloat32 = 7;                       // ncclFloat32 in ncclDataType_t

using GetUniqueIdFn = int (*)(NcclUniqueId*);
using CommInitRankFn = int (*)(NcclComm**, int, NcclUniqueId, int);
using AllGatherFn = int (*)(const void*, void*, size_t, int, NcclComm*, cudaStream_t);
using CommDestroyFn = int (*)(NcclComm*);
using GetErrorStringFn = const char* (*)(int);

struct Comm {
    void* dl = nullptr;
    GetUniqueIdFn get_unique_id = nullptr;
    CommInitRankFn init_rank = nullptr;
    AllGatherFn all_gather = nullptr;
    CommDestroyFn destroy = nullptr;
    GetErrorStringFn error_string = nullptr;
    NcclComm* comm = nullptr;
    int rank = 0, world = 1;
};

Comm& comm() { static Comm c; return c; }

bool bind_nccl() {
    Comm& c = comm();
    if (c.dl) return true;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return fail("comm: libnccl.so.2 cannot be loaded: %s", dlerror());
    c.get_unique_id = (GetUniqueIdFn)dlsym(h, "ncclGetUniqueId");
    c.init_rank = (CommInitRankFn)dlsym(h, "ncclCommInitRank");
    c.all_gather = (AllGatherFn)dlsym(h, "ncclAllGather");
    c.destroy = (CommDestroyFn)dlsym(h, "ncclCommDestroy");
    c.error_string = (GetErrorStringFn)dlsym(h, "ncclGetErrorString");
    if (!c.get_unique_id || !c.init_rank || !c.all_gather || !c.destroy || !c.error_string) {
        dlclose(h);
        return fail("comm: libnccl.so.2 lacks an expected symbol");
    }
    c.dl = h;
    return true;
}

bool nccl_ok(int rc, const char* where) {
    if (rc == 0) return true;
    return fail("comm: %s: %s", where, comm().error_string ? comm().error_string(rc) : "NCCL error");
}

}  // namespace
}  // namespace tmc

using namespace tmc;

extern "C" {

size_t tm_cuda_comm_id_bytes(void) { return sizeof(NcclUniqueId); }

bool tm_cuda_comm_unique_id(void* out) {
    if (!out) return fail("comm: null id buffer");
    if (!bind_nccl()) return false;
    NcclUniqueId id;
    if (!nccl_ok(comm().get_unique_id(&id), "ncclGetUniqueId")) return false;
    std::memcpy(out, &id, sizeof id);
    return true;
}

bool tm_cuda_comm_init(int rank, int world, const void* id_bytes) {
    if (!ensure_init(-1)) return false;
    Comm& c = comm();
    if (c.comm) return fail("comm: already initialised");
    if (world < 1 || rank < 0 || rank >= world) return fail("comm: rank %d of %d is not valid", rank, world);
    if (world == 1) { c.rank = 0; c.world = 1; return true; }
    if (!id_bytes) return fail("comm: null id");
    if (!bind_nccl()) return false;
    NcclUniqueId id;
    std::memcpy(&id, id_bytes, sizeof id);
    if (!nccl_ok(c.init_rank(&c.comm, world, id, rank), "ncclCommInitRank")) { c.comm = nullptr; return false; }
    c.rank = rank; c.world = world;
    return true;
}

int tm_cuda_comm_rank(void) { return comm().rank; }
int tm_cuda_comm_world(void) { return comm().world; }

bool tm_cuda_comm_destroy(void) {
    Comm& c = comm();
    if (!c.comm) { c.rank = 0; c.world = 1; return true; }
    State& s = state();
    if (s.ready) {
        cudaStreamSynchronize(s.stream);
        tm_cuda_tok_graph_destroy(-1);                 // every graph: they may hold the communicator
    }
    const bool ok = nccl_ok(c.destroy(c.comm), "ncclCommDestroy");
    c.comm = nullptr; c.rank = 0; c.world = 1;
    return ok;
}

// dst[dst_off + r * count .. + count) of every rank <- src[src_off .. + count) of rank r, fp32.
// In place when src is the caller's own slice of dst (src_off == dst_off + rank * count * 4).
void tm_cuda_tok_all_gather(int srcslot, size_t src_off, int dstslot, size_t dst_off, unsigned count) {
    if (!ensure_init(-1)) return;
    State& s = state();
    Comm& c = comm();
    auto latch = [&](const char* msg) { fail("tok_all_gather: %s", msg); s.sticky = true; };
    if (!count) return latch("empty gather");
    if (src_off % 16 || dst_off % 16 || ((size_t)count * 4) % 16) return latch("offsets and per-rank bytes must be multiples of 16");
    const size_t per = (size_t)count * 4;
    if (srcslot < 0 || dstslot < 0 || srcslot >= (int)s.slots.size() || dstslot >= (int)s.slots.size()) return latch("unknown slot");
    const Slot& a = s.slots[srcslot];
    const Slot& b = s.slots[dstslot];
    if (!a.ptr || a.bytes < src_off + per) return latch("source slot is too small");
    if (!b.ptr || b.bytes < dst_off + per * (size_t)c.world) return latch("destination slot is too small");
    const uint8_t* src = a.ptr + src_off;
    uint8_t* dst = b.ptr + dst_off;
    uint8_t* mine = dst + per * (size_t)c.rank;
    const bool in_place = src == mine;
    if (!in_place && src < dst + per * (size_t)c.world && dst < src + per) return latch("source overlaps the gathered range without being this rank's slice");
    if (c.world == 1) {
        if (!in_place && cudaMemcpyAsync(dst, src, per, cudaMemcpyDeviceToDevice, s.stream) != cudaSuccess) { check_launch("tok_all_gather"); s.sticky = true; }
        return;
    }
    if (!c.comm) return latch("no communicator: call tm_cuda_comm_init first");
    if (!nccl_ok(c.all_gather(src, dst, count, kNcclFloat32, c.comm, s.stream), "ncclAllGather")) s.sticky = true;
}

}  // extern "C"
