// tests/host/lane_emul.cpp — runs the GEMV lane maps (gemv_lanes.cuh) on the CPU.
//
// The streaming GEMV kernel splits every step of a weight row over 32 lanes; which
// bytes and which activations a lane touches is pure index arithmetic that can be
// wrong without any GPU being involved. This harness replays that arithmetic lane
// by lane with the host versions of the same inline functions: it stages x exactly
// as the kernel does (swizzled float4 slots, per-32-block sums), walks the steps of
// each row, and adds the 32 lane partials in the kernel's butterfly order. The test
// suite compares the result with the CPU checker, so a wrong lane map is caught
// before the kernel is ever launched.
#include "../../tensormark_b200/csrc/gemv_lanes.cuh"

#include <algorithm>
#include <cstdlib>
#include <vector>

using namespace tmc;

template <int DT>
static void emul(const uint8_t* W, const float* x, float* y, unsigned N, unsigned K, unsigned row_bytes) {
    using L = Lane<DT>;
    const unsigned nchunks = (K + L::STEP_W - 1) / L::STEP_W, kpad = nchunks * L::STEP_W;
    std::vector<float4> xs4(kpad / 4);
    std::vector<float> xsum(kpad / 32, 0.f);
    for (unsigned q = 0; q < kpad / 4; ++q) {
        float4 v = {0.f, 0.f, 0.f, 0.f};
        if (q * 4 < K) { v.x = x[4 * q]; v.y = x[4 * q + 1]; v.z = x[4 * q + 2]; v.w = x[4 * q + 3]; }
        xs4[x_slot(q)] = v;
    }
    for (unsigned b = 0; b < K / 32; ++b) {
        float s = 0.f;
        for (int i = 0; i < 8; ++i) { const float* v = x + b * 32 + 4 * i; s += (v[0] + v[1]) + (v[2] + v[3]); }
        xsum[b] = s;
    }
    // a stage as the kernel sees it: 16-byte aligned, garbage beyond the valid bytes
    std::vector<uint8_t> stage_raw(L::STEP_BYTES + 64, 0xA5);
    uint8_t* stage = stage_raw.data() + ((16 - ((uintptr_t)stage_raw.data() & 15)) & 15);
    for (unsigned row = 0; row < N; ++row) {
        float lane_acc[32] = {0};
        for (unsigned c = 0; c < nchunks; ++c) {
            const unsigned off = c * L::STEP_BYTES, bytes = std::min<unsigned>(L::STEP_BYTES, row_bytes - off);
            std::fill(stage, stage + L::STEP_BYTES, 0xA5);
            memcpy(stage, W + (size_t)row * row_bytes + off, bytes);
            const unsigned wchunk = std::min<unsigned>(L::STEP_W, K - c * L::STEP_W);
            const int units = (int)(wchunk / L::UNIT_W);
            for (int lane = 0; lane < 32; ++lane) {
                typename L::X xr;
                L::load_x(xr, xs4.data(), xsum.data(), (int)c, lane);
                int valid = units;
                if (L::LANE_UNITS == 2) { valid = std::max(0, std::min(2, units - 2 * lane)); if (!valid) continue; }
                lane_acc[lane] += L::dot(stage + (L::LANE_UNITS == 2 ? lane * L::LANE_BYTES : 0), xr, lane, valid);
            }
        }
        float v[32];
        for (int l = 0; l < 32; ++l) v[l] = lane_acc[l];
        for (int o = 16; o; o >>= 1) { float t[32]; for (int l = 0; l < 32; ++l) t[l] = v[l] + v[l ^ o]; memcpy(v, t, sizeof v); }
        y[row] = v[0];
    }
}

extern "C" __attribute__((visibility("default")))
int lane_emul_gemv(int dtype, const void* W, const float* x, float* y, unsigned N, unsigned K) {
    const unsigned be = (dtype == 5 || dtype == 6) ? 256 : 32;
    const unsigned bb = dtype == 0 ? 34 : dtype == 1 ? 18 : dtype == 4 ? 20 : dtype == 5 ? 176 : 210;
    if (K % be) return 0;
    const unsigned rb = K / be * bb;
    switch (dtype) {
        case 0: emul<0>((const uint8_t*)W, x, y, N, K, rb); return 1;
        case 1: emul<1>((const uint8_t*)W, x, y, N, K, rb); return 1;
        case 4: emul<4>((const uint8_t*)W, x, y, N, K, rb); return 1;
        case 5: emul<5>((const uint8_t*)W, x, y, N, K, rb); return 1;
        case 6: emul<6>((const uint8_t*)W, x, y, N, K, rb); return 1;
        default: return 0;
    }
}
