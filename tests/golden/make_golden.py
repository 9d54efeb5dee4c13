"""Generate the golden vectors of the block formats from the REFERENCE's own code.

Run in a checkout where the reference tree is present and oracle/_ref/libtm_ref.so
was built from it (`make -C oracle`): every expected value below is produced by the
reference's tmq::dequantize_row_* / quantize_row_* / fp16 conversions (quant.h),
not by this repository's restatement. The output, tests/golden/blocks.npz, is
committed; tests compare the restated oracle, the host header and the CUDA kernels
against it bit for bit.

    python tests/golden/make_golden.py
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import binding  # noqa: E402
from tensormark_b200 import synth  # noqa: E402

SPECIAL_HALVES = [0x0000, 0x8000, 0x0001, 0x03ff, 0x0400, 0x8001, 0x3c00, 0xbc00, 0x7bff, 0x7c00, 0xfc00, 0x7e00, 0x7c01, 0x1234]


def special_blocks(dtype: int, rng: np.random.Generator) -> np.ndarray:
    """One block per special scale encoding (zero, subnormal, max, inf, NaN ...) with random codes,
    plus all-min / all-max code blocks."""
    bb = synth.BLOCK_BYTES[dtype]
    scale_off = {0: [0], 1: [0], 4: [0, 2], 5: [0, 2], 6: [208], 7: [0], 8: [0, 2]}[dtype]
    out = []
    for h in SPECIAL_HALVES:
        for off in scale_off:
            b = rng.integers(0, 256, size=bb, dtype=np.uint8)
            # keep the other scale ordinary so only one field is special at a time
            for o2 in scale_off:
                b[o2:o2 + 2] = np.array([0x2400 & 0xff, 0x2400 >> 8], dtype=np.uint8)
            b[off:off + 2] = np.array([h & 0xff, h >> 8], dtype=np.uint8)
            out.append(b)
    for fill in (0x00, 0xff, 0x0f, 0xf0, 0x80, 0x7f):
        b = np.full(bb, fill, dtype=np.uint8)
        for o2 in scale_off:
            b[o2:o2 + 2] = np.array([0x00, 0x2c], dtype=np.uint8)   # 0x2c00 = 0.0625
        out.append(b)
    return np.stack(out)


def main() -> None:
    ref = binding.reference()
    if ref is None:
        raise SystemExit("oracle/_ref/libtm_ref.so is missing: run `make -C oracle` where the reference tree exists")
    out = {}
    rng = np.random.Generator(np.random.Philox(key=[2026, 7]))
    # the formats quant.h itself dequantizes, TQ2 last (so the earlier formats' vectors do not depend on it). GGUF's own
    # Q4_0 (dtype 9) is decoded in llama.h, not quant.h: it is pinned by its relation to Q4_0 instead (tests/test_oracle.py).
    for dt in (synth.Q8_0, synth.Q4_0, synth.Q4_1, synth.Q5_K, synth.Q6_K, synth.Q4_K, synth.TQ2):
        name = synth.DTYPE_NAMES[dt]
        be = synth.BLOCK_ELEMS[dt]
        k = 512
        blocks = synth.make_weights(dt, 6, k, seed=100 + dt).reshape(-1, synth.BLOCK_BYTES[dt])
        blocks = np.concatenate([blocks, special_blocks(dt, rng)])
        n = blocks.shape[0] * be
        deq = ref.dequant(dt, blocks, n)
        out[f"{name}_blocks"] = blocks
        out[f"{name}_dequant_bits"] = deq.view(np.uint32)
    # the reference's own quantizers on seeded floats: realistic scales, every code reachable
    x = (rng.standard_normal(32 * 64) * np.repeat(np.exp(rng.standard_normal(64) * 3.0), 32)).astype(np.float32)
    for dt in (0, 1, 7):
        q = ref.quantize(dt, x)
        out[f"{synth.DTYPE_NAMES[dt]}_quantized_from"] = x
        out[f"{synth.DTYPE_NAMES[dt]}_quantized_blocks"] = q
        out[f"{synth.DTYPE_NAMES[dt]}_quantized_dequant_bits"] = ref.dequant(dt, q, x.size).view(np.uint32)
    # fp16 conversions: every half, and floats around every rounding boundary
    halves = np.arange(65536, dtype=np.uint32)
    out["fp16_to_fp32_bits"] = np.array([np.float32(ref.lib.tmref_fp16_to_fp32(int(h))).view(np.uint32) for h in halves], dtype=np.uint32)
    fl = np.concatenate([
        rng.standard_normal(4096).astype(np.float32) * np.float32(1e-4),
        rng.standard_normal(4096).astype(np.float32),
        (rng.standard_normal(2048) * 7e4).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.99, 65520.0, 6.1e-5, 5.96e-8, 2.98e-8, 2.9802325e-8, 1e-10, np.inf, -np.inf, np.nan], dtype=np.float32),
        (halves[::7].astype(np.uint32) << 13).view(np.float32)[:2048],
    ])
    out["fp32_to_fp16_in_bits"] = fl.view(np.uint32)
    out["fp32_to_fp16_out"] = np.array([ref.lib.tmref_fp32_to_fp16(float(v)) if not np.isnan(v) else ref.lib.tmref_fp32_to_fp16(float("nan")) for v in fl], dtype=np.uint16)
    path = os.path.join(ROOT, "tests", "golden", "blocks.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
