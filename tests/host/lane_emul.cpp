// tests/host/lane_emul.cpp — runs the GEMV lane maps (gemv_lanes.cuh) on the CPU.
//
// The streaming GEMV kernel splits every step of a weight row over 32 lanes; which
// bytes and which activations a lane touches is pure index arithmetic that can be
// wrong without any GPU being involved. This harness replays that arithmetic lane
// by lane with the host versions of the same inline functions: it stages x exactly
// as the kernel does (block floating point planes scattered into the lanes' x
// units), walks the steps of each row, and adds the 32 lane partials in the kernel's
// butterfly order. The test
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
    const unsigned nchunks = (K + L::STEP_W - 1) / L::STEP_W, nunits = nchunks * 32;
    // x units exactly as the kernel stages them: zero fill, then per 32-block the scale, the
    // run sums and every activation's plane bytes
    std::vector<uint32_t> units((size_t)nunits * L::XW, 0u);
    for (unsigned b = 0; b < K / 32; ++b) {
        float v[32], amax = 0.f;
        bool bad = false;
        for (int i = 0; i < 32; ++i) { v[i] = x[b * 32 + i]; const float a = fabsf(v[i]); bad = bad || !(a <= 3.0e38f); amax = a > amax ? a : amax; }
        float inv;
        const float sc = block_scale(amax, bad, inv);
        float s8[4], s16[2], s32;
        for (int g = 0; g < 4; ++g) { float t = 0.f; for (int i = 0; i < 8; ++i) t += v[8 * g + i]; s8[g] = t; }
        s16[0] = s8[0] + s8[1]; s16[1] = s8[2] + s8[3]; s32 = s16[0] + s16[1];
        for (int lane = 0; lane < 32; ++lane) {
            int8_t q[kPlanes];
            quantize_elem(v[lane], inv, q);
            for (int t = 0; t < kPlanes; ++t) reinterpret_cast<int8_t*>(units.data())[L::plane_byte(b * 32 + lane, t)] = q[t];
            L::scalars(units.data(), b, lane, (lane & 3) ? 99 : lane / 4, sc, s8[lane / 8], s16[lane / 16], s32);
        }
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
            const int nu = (int)(wchunk / L::UNIT_W);
            for (int lane = 0; lane < 32; ++lane) {
                typename L::X xr;
                load_x_unit<DT>(xr, units.data(), c * 32 + lane);
                int valid = nu;
                if (L::LANE_UNITS == 2) { valid = std::max(0, std::min(2, nu - 2 * lane)); if (!valid) continue; }
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
    const unsigned be = (dtype == 5 || dtype == 6 || dtype == 8) ? 256 : 32;
    const unsigned bb = dtype == 0 ? 34 : (dtype == 1 || dtype == 9) ? 18 : dtype == 4 ? 20 : dtype == 5 ? 176 : dtype == 8 ? 144 : 210;
    if (K % be) return 0;
    const unsigned rb = K / be * bb;
    switch (dtype) {
        case 0: emul<0>((const uint8_t*)W, x, y, N, K, rb); return 1;
        case 1: emul<1>((const uint8_t*)W, x, y, N, K, rb); return 1;
        case 4: emul<4>((const uint8_t*)W, x, y, N, K, rb); return 1;
        case 5: emul<5>((const uint8_t*)W, x, y, N, K, rb); return 1;
        case 6: emul<6>((const uint8_t*)W, x, y, N, K, rb); return 1;
        case 8: emul<8>((const uint8_t*)W, x, y, N, K, rb); return 1;
        case 9: emul<9>((const uint8_t*)W, x, y, N, K, rb); return 1;
        default: return 0;
    }
}
