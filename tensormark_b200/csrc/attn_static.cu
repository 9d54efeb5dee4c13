// attn_static.cu — decode attention with its split-K scratch in a static device array.
//
// tm_cuda_attn_decode_dev needs a caller-provided scratch buffer for the per-split partial
// outputs and softmax statistics. Some callers cannot provide one: a serving engine that has
// already handed every free byte of device memory to its own pool (a cudaMalloc there simply
// fails), or a latency-critical loop that must not pay cudaMalloc's implicit device-wide
// synchronisation. For them this file offers one more entry point that allocates nothing: the
// scratch is a file-scope array that every GPU loading the library carries until the process
// exits (kStaticScratchBytes, 512 KiB per GPU).
//
// Host code must not pass the array's NAME to a kernel: in host code that name is only a
// stand-in for the symbol, not a device address. The device address is looked up once per
// device with cudaGetSymbolAddress, with that device current, and cached.
#include "cuda_shim.h"
#include "common.cuh"
#include "glue.h"

#include <atomic>
#include <cmath>

namespace tmc {
namespace {

constexpr size_t kStaticScratchBytes = TM_CUDA_ATTN_STATIC_SCRATCH_BYTES;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) float g_attn_scratch[kStaticScratchBytes / sizeof(float)];

struct PerDevice {
    std::atomic<float*> scratch{nullptr};   // device address of g_attn_scratch on this device; published last
    int sms = 0;
};
PerDevice g_dev[kMaxDevices];

// Resolve the array's address on the current device (first call on that device only). Two host threads that make
// their first call at once both look the address up and store the same two values; the address is stored last with
// release order, so whoever reads it non-null also reads the SM count.
PerDevice* current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { fail("attn_decode_static: no current CUDA device"); return nullptr; }
    PerDevice& d = g_dev[dev];
    if (!d.scratch.load(std::memory_order_acquire)) {
        float* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void**)&p, g_attn_scratch);
        if (e != cudaSuccess || !p) { fail("attn_decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e)); return nullptr; }
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) { fail("attn_decode_static: cannot read the SM count"); return nullptr; }
        d.sms = sms;
        d.scratch.store(p, std::memory_order_release);
    }
    return &d;
}

}  // namespace
}  // namespace tmc

using namespace tmc;

extern "C" bool tm_cuda_attn_decode_static_dev(const float* q, const void* kc, const void* vc, float* out, unsigned H,
                                               unsigned KVH, unsigned dh, unsigned ctx, unsigned allow, float scale,
                                               int kv_half, void* stream) {
    if (!q || !kc || !vc || !out) return fail("attn_decode_static: null pointer");
    if (!H || !KVH || !dh || !ctx || !allow || allow > ctx || H % KVH || !std::isfinite(scale) || scale <= 0)
        return fail("attn_decode_static: invalid decode attention dimensions or scale");
    PerDevice* d = current_device();
    if (!d) return false;
    const unsigned REP = H / KVH;
    if (dh != 64 && dh != 128) return fail("attn_decode_static: head dimension %u (64 and 128 are built)", dh);
    if (REP != 1 && REP != 2 && REP != 4 && REP != 8) return fail("attn_decode_static: %u query heads per K/V head (1, 2, 4 or 8)", REP);
    // The allocating entry's split rule (one helper for both): enough (kv head, split) CTAs to cover the GPU, at
    // least 32 positions per split. The static array must hold all of them; a shape that needs more is refused rather
    // than run with fewer splits.
    const AttnPlan pl = plan_attention_sms((unsigned)d->sms, H, KVH, dh, ctx, allow, (size_t)1 << 40);
    const size_t need = (size_t)pl.nsplit * H * (dh + 2) * sizeof(float);
    if (need > kStaticScratchBytes)
        return fail("attn_decode_static: this shape needs %zu bytes of split-K scratch, the static array holds %zu; "
                    "use tm_cuda_attn_decode_dev with a buffer of your own", need, kStaticScratchBytes);
    // Nothing has to be cleared: every word the combine pass reads was written by the split
    // pass of this same call.
    return launch_attention(q, kc, vc, kv_half != 0, d->scratch.load(std::memory_order_acquire), out, H, KVH, dh, ctx, allow, scale, REP, pl,
                            (cudaStream_t)stream);
}
