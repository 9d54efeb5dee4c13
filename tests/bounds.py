"""Derived error bound of the streaming GEMV's activation format (no GPU needed).

The kernel rounds every activation once to a multiple of s / 128 with s = max|x| / 127 over its 32-block (two
signed 8-bit digits; tensormark_b200/csrc/gemv_lanes.cuh), so |x_i - x~_i| <= max|x_block| / (127 * 256) and
an output can be off by at most

    sum over blocks of  max|x_block| / 32512 * sum_{i in block} |w_i|

before fp32 accumulation noise (a few 1e-7 * sum|w x|). For activations of one scale this is about
9e-5 * sum|w x| in the worst alignment of rounding errors and a few 1e-6 in practice; the contract of the path
is 1e-3 * sum|w x|."""
from __future__ import annotations

import numpy as np

PLANE_STEP = 1.0 / (127.0 * 256.0)


def activation_rounding_bound(orc, dt: int, W: np.ndarray, x: np.ndarray, n: int, k: int) -> np.ndarray:
    """Per-output bound described above, float64 [n]."""
    w = np.abs(orc.dequant(dt, W, n * k).astype(np.float64)).reshape(n, k // 32, 32).sum(2)
    bmax = np.abs(np.asarray(x, np.float64).reshape(-1, 32)).max(1)
    return (w * bmax[None, :]).sum(1) * PLANE_STEP
