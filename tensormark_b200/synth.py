"""Seeded synthetic block-quantized weights and activations.

The benchmark configurations are fully synthetic: each names a block format, a
shape, a seed and the distribution of every field of a block. This module is the
single generator that the tests, the smoke check and the benchmark share, so the
CPU checker and the CUDA path always see identical bytes.

Block layouts are the serialized ones of the reference (tensormark/quant.h:35-49,
214-249); dtype ids follow tensormark/tmq.h:48-60.
"""
from __future__ import annotations

import numpy as np

Q8_0, Q4_0, F16, Q4_1, Q5_K, Q6_K, TQ2, Q4_K, GGUF_Q4_0, BF16 = 0, 1, 3, 4, 5, 6, 7, 8, 9, 10
DTYPE_NAMES = {Q8_0: "Q8_0", Q4_0: "Q4_0", Q4_1: "Q4_1", Q5_K: "Q5_K", Q6_K: "Q6_K", TQ2: "TQ2", Q4_K: "Q4_K", GGUF_Q4_0: "GGUF_Q4_0"}
BLOCK_ELEMS = {Q8_0: 32, Q4_0: 32, Q4_1: 32, Q5_K: 256, Q6_K: 256, TQ2: 128, Q4_K: 256, GGUF_Q4_0: 32}
BLOCK_BYTES = {Q8_0: 34, Q4_0: 18, Q4_1: 20, Q5_K: 176, Q6_K: 210, TQ2: 34, Q4_K: 144, GGUF_Q4_0: 18}


def weight_bytes(dtype: int, n_out: int, n_in: int) -> int:
    """Payload bytes of an n_out x n_in tensor (tensormark/tmq.h:124-133)."""
    be = BLOCK_ELEMS[dtype]
    if n_in % be:
        raise ValueError("row width is not whole blocks")
    return n_out * (n_in // be) * BLOCK_BYTES[dtype]


def gemv_bytes(dtype: int, n_out: int, n_in: int) -> int:
    """Algorithmic bytes of one GEMV: the weight payload plus x and y in fp32."""
    return weight_bytes(dtype, n_out, n_in) + 4 * n_in + 4 * n_out


def rng_for(seed: int, stream: int = 0) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[seed, stream]))


def _half_bytes(values: np.ndarray) -> np.ndarray:
    """fp32 -> IEEE half (round to nearest even) -> little-endian byte pairs."""
    return values.astype(np.float32).astype(np.float16).view(np.uint8).reshape(-1, 2)


def make_weights(dtype: int, n_out: int, n_in: int, seed: int, stream: int = 1) -> np.ndarray:
    """Random blocks for an n_out x n_in tensor as a uint8 array [n_out, row_bytes].

    Field distributions:
      Q4_0  d = half(|N(0,1)| * 0.02), 32 codes uniform in 0..15
      Q8_0  d = half(|N(0,1)| * 0.005), 32 int8 codes uniform in -127..127
      Q4_1  d = half(|N(0,1)| * 0.02), m = half(N(0, 0.05)), codes uniform in 0..15
      Q5_K  d, dmin = half(|N(0,1)| * 0.001); scales, qh, qs uniform random bytes
      Q6_K  ql, qh uniform bytes; scales int8 uniform in -32..31; d = half(|N(0,1)| * 0.001)
      Q4_K  d, dmin = half(|N(0,1)| * 0.001); scales, qs uniform random bytes
    """
    g = rng_for(seed, stream)
    nb = n_out * (n_in // BLOCK_ELEMS[dtype])
    bb = BLOCK_BYTES[dtype]
    out = np.empty((nb, bb), dtype=np.uint8)
    if dtype in (Q4_0, GGUF_Q4_0):               # the same bytes; the two formats differ in which element a nibble is
        out[:, 0:2] = _half_bytes(np.abs(g.standard_normal(nb)) * 0.02)
        out[:, 2:18] = g.integers(0, 256, size=(nb, 16), dtype=np.uint8)
    elif dtype == Q8_0:
        out[:, 0:2] = _half_bytes(np.abs(g.standard_normal(nb)) * 0.005)
        out[:, 2:34] = g.integers(-127, 128, size=(nb, 32), dtype=np.int8).view(np.uint8)
    elif dtype == Q4_1:
        out[:, 0:2] = _half_bytes(np.abs(g.standard_normal(nb)) * 0.02)
        out[:, 2:4] = _half_bytes(g.standard_normal(nb) * 0.05)
        out[:, 4:20] = g.integers(0, 256, size=(nb, 16), dtype=np.uint8)
    elif dtype == Q5_K:
        out[:, 0:2] = _half_bytes(np.abs(g.standard_normal(nb)) * 0.001)
        out[:, 2:4] = _half_bytes(np.abs(g.standard_normal(nb)) * 0.001)
        out[:, 4:176] = g.integers(0, 256, size=(nb, 172), dtype=np.uint8)
    elif dtype == Q4_K:
        out[:, 0:2] = _half_bytes(np.abs(g.standard_normal(nb)) * 0.001)
        out[:, 2:4] = _half_bytes(np.abs(g.standard_normal(nb)) * 0.001)
        out[:, 4:144] = g.integers(0, 256, size=(nb, 140), dtype=np.uint8)
    elif dtype == TQ2:                            # d = half(|N(0,1)| * 0.02), 128 codes uniform in 0..3 (3 = +2 never comes out of the
        out[:, 0:2] = _half_bytes(np.abs(g.standard_normal(nb)) * 0.02)      # reference's quantizer but must decode, quant.h:489-492)
        out[:, 2:34] = g.integers(0, 256, size=(nb, 32), dtype=np.uint8)
    elif dtype == Q6_K:
        out[:, 0:192] = g.integers(0, 256, size=(nb, 192), dtype=np.uint8)
        out[:, 192:208] = g.integers(-32, 32, size=(nb, 16), dtype=np.int8).view(np.uint8)
        out[:, 208:210] = _half_bytes(np.abs(g.standard_normal(nb)) * 0.001)
    else:
        raise ValueError(f"no block generator for dtype {dtype}")
    return out.reshape(n_out, -1)


def make_activations(shape, seed: int, stream: int = 2) -> np.ndarray:
    """fp32 N(0,1) activations."""
    return rng_for(seed, stream).standard_normal(shape, dtype=np.float32)


def make_tokens(n: int, vocab: int, seed: int, stream: int = 3) -> np.ndarray:
    return rng_for(seed, stream).integers(0, vocab, size=n, dtype=np.uint32)


# TinyLlama-1.1B and Llama-3-8B projection shapes (out, in) used by the sweeps.
TINYLLAMA_SHAPES = [(2048, 2048), (256, 2048), (5632, 2048), (2048, 5632), (32000, 2048)]
LLAMA3_8B_SHAPES = [(4096, 4096), (14336, 4096), (4096, 14336)]


# ---- synthetic Llama-style models (random-init weights of a named architecture) -----------
LLAMA3_8B = dict(L=32, D=4096, H=32, KVH=8, dh=128, F=14336, V=128256, ctx=1024, theta=500000.0, eps=1e-5,
                 dt_proj=Q4_0, dt_head=Q6_K, dt_embed=Q4_0)
TINY_CHAIN = dict(L=2, D=256, H=4, KVH=2, dh=64, F=512, V=1024, ctx=96, theta=500000.0, eps=1e-5,
                  dt_proj=Q4_0, dt_head=Q6_K, dt_embed=Q4_0)


def make_llama(cfg: dict, seed: int, progress=None) -> dict:
    """Random-init weights for a Llama-style decoder, every block tensor inside ONE contiguous
    uint8 blob (as tensors sit in a mapped .tmq file), 16-byte aligned. Returns
    {"blob": uint8 array, "<name>": view, ...} with names embed, head, rmsf, l{i}.q/k/v/o/gate/up/down/rms1/rms2.
    Block contents follow the per-format distributions of make_weights; norm weights are N(1, 0.02)."""
    L, D, F, V = cfg["L"], cfg["D"], cfg["F"], cfg["V"]
    QD, KVD = cfg["H"] * cfg["dh"], cfg["KVH"] * cfg["dh"]
    specs = [("embed", cfg["dt_embed"], V, D), ("head", cfg["dt_head"], V, D)]
    for l in range(L):
        for name, n, k in (("q", QD, D), ("k", KVD, D), ("v", KVD, D), ("o", D, QD), ("gate", F, D), ("up", F, D), ("down", D, F)):
            specs.append((f"l{l}.{name}", cfg["dt_proj"], n, k))
    offs, cur = {}, 0
    for name, dt, n, k in specs:
        offs[name] = cur
        cur += (weight_bytes(dt, n, k) + 15) // 16 * 16
    blob = np.zeros(cur + 64, dtype=np.uint8)
    out = {"blob": blob}
    for i, (name, dt, n, k) in enumerate(specs):
        nb = weight_bytes(dt, n, k)
        view = blob[offs[name]: offs[name] + nb].reshape(n, -1)
        # large tensors are generated in row slabs to bound the temporary memory
        step = max(1, (64 << 20) // max(1, nb // n))
        for r0 in range(0, n, step):
            r1 = min(n, r0 + step)
            view[r0:r1] = make_weights(dt, r1 - r0, k, seed, stream=1000 + 64 * i + r0 // step)
        out[name] = view
        if progress:
            progress(name)
    g = rng_for(seed, 7)
    out["rmsf"] = (1.0 + 0.02 * g.standard_normal(D)).astype(np.float32)
    for l in range(L):
        out[f"l{l}.rms1"] = (1.0 + 0.02 * g.standard_normal(D)).astype(np.float32)
        out[f"l{l}.rms2"] = (1.0 + 0.02 * g.standard_normal(D)).astype(np.float32)
    return out
