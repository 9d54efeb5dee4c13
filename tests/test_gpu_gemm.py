"""GPU parity of the tensor-core prefill GEMM: sampled outputs within 1e-3 * sum|a w| of the fp64 reference."""
from __future__ import annotations

import numpy as np
import pytest

from tensormark_b200 import lib, synth
from tests.gpu_util import dev_bytes, dev_f32, ptr, stream_ptr

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _gemm_dev(cuda, torch, dt, W, A, m, n, k):
    Wd, Ad = dev_bytes(torch, W), dev_f32(torch, A)
    Cd = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    need = cuda.tm_cuda_sgemm_q_workspace(m, n, k, dt)
    ws = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
    base = (ws.data_ptr() + 255) // 256 * 256
    import ctypes as C
    lib.check(cuda.tm_cuda_sgemm_q_dev(ptr(Ad), ptr(Wd), ptr(Cd), m, n, k, dt, C.c_void_p(base), need, stream_ptr(torch)),
              "tm_cuda_sgemm_q_dev")
    torch.cuda.synchronize()
    return Cd.cpu().numpy()


def _check_samples(orc, dt, W, A, Cm, n, k, ns=4096, seed=0):
    rng = np.random.default_rng(seed)
    m = A.shape[0]
    idx = np.stack([rng.integers(0, m, ns), rng.integers(0, n, ns)], axis=1).astype(np.int32)
    # always include the corners and the last partial tiles
    idx[:4] = [[0, 0], [m - 1, n - 1], [0, n - 1], [m - 1, 0]]
    y64, yabs = orc.gemm_f64_samples(dt, W, A, n, k, idx)
    got = Cm[idx[:, 0], idx[:, 1]]
    assert not np.isnan(got).any()
    err = np.abs(got - y64)
    assert np.all(err <= TOL * yabs), float((err / yabs).max())


@pytest.mark.parametrize("dt,m,n,k", [
    (synth.Q4_0, 64, 256, 512),        # one tile, short K
    (synth.Q4_0, 40, 256, 512),        # a 48-token tile: the last 32-column read of the accumulator is half stale
    (synth.Q4_0, 7, 128, 64),          # the narrowest tile, one k-block
    (synth.Q4_0, 300, 384, 2048),      # ragged token tile
    (synth.Q4_0, 257, 130, 96),        # ragged in both, K not a multiple of 64
    (synth.Q6_K, 100, 256, 1024),
    (synth.Q4_0, 500, 640, 320),       # two and a half pairs of row tiles, five k-blocks
    (synth.Q8_0, 50, 128, 256),
    (synth.Q4_1, 50, 128, 256),
    (synth.Q5_K, 50, 128, 512),
    (synth.Q4_K, 50, 128, 512),
])
def test_small_shapes_full_check(cuda, torch_mod, orc, dt, m, n, k):
    W = synth.make_weights(dt, n, k, seed=4)
    A = synth.make_activations((m, k), seed=4)
    Cm = _gemm_dev(cuda, torch_mod, dt, W, A, m, n, k)
    ref = orc.gemm(dt, W, A, m, n, k, threads=4)
    # the fp32 CPU GEMM is itself within 1e-5 of fp64; compare every element against it at the path's bar
    absum = np.abs(A) @ np.abs(orc.dequant(dt, W, n * k).reshape(n, k)).T
    assert np.all(np.abs(Cm - ref) <= TOL * absum)


@pytest.mark.parametrize("dt,n,k", [(synth.Q4_0, 5632, 2048), (synth.Q4_0, 2048, 5632), (synth.Q6_K, 32000, 2048)])
def test_config4_prefill_shapes_sampled(cuda, torch_mod, orc, dt, n, k):
    m = 2000
    W = synth.make_weights(dt, n, k, seed=4)
    A = synth.make_activations((m, k), seed=4)
    Cm = _gemm_dev(cuda, torch_mod, dt, W, A, m, n, k)
    _check_samples(orc, dt, W, A, Cm, n, k)


def test_host_pointer_entries(cuda, orc):
    m, k = 40, 512
    ns = [128, 64, 96]
    Ws = [synth.make_weights(synth.Q4_0, n, k, seed=70 + i) for i, n in enumerate(ns)]
    A = synth.make_activations((m, k), seed=7)
    import ctypes as C
    Cm = np.empty((m, sum(ns)), np.float32)
    ptrs = (C.c_void_p * 3)(*[w.ctypes.data for w in Ws])
    cn = (C.c_uint * 3)(*ns)
    lib.check(cuda.tm_cuda_q4_prefill(A.ctypes.data, ptrs, cn, 3, Cm.ctypes.data, m, k), "tm_cuda_q4_prefill")
    col = 0
    for w, n in zip(Ws, ns):
        ref = orc.gemm(synth.Q4_0, w, A, m, n, k)
        absum = np.abs(A) @ np.abs(orc.dequant(synth.Q4_0, w, n * k).reshape(n, k)).T
        assert np.all(np.abs(Cm[:, col: col + n] - ref) <= TOL * absum)
        col += n
    C1 = np.empty((m, ns[0]), np.float32)
    lib.check(cuda.tm_cuda_sgemm_q4(A.ctypes.data, Ws[0].ctypes.data, C1.ctypes.data, m, ns[0], k), "tm_cuda_sgemm_q4")
    assert np.array_equal(C1.view(np.uint32), np.ascontiguousarray(Cm[:, : ns[0]]).view(np.uint32))
    assert not cuda.tm_cuda_sgemm_q4(A.ctypes.data, Ws[0].ctypes.data, C1.ctypes.data, m, ns[0], 500)
    cuda.tm_cuda_release_weights()


def test_q4_kernel_with_in_kernel_dequant(torch_mod):
    """The Q4_0 GEMM whose producer warps dequantize the blocks into the shared-memory tiles (selected with
    TM_GEMM_FUSED=1 at first use, hence a fresh process): the same checks as the default path."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, TM_GEMM_FUSED="1")
    sel = "test_small_shapes_full_check or (test_config4_prefill_shapes_sampled and not 32000)"
    r = subprocess.run([sys.executable, "-m", "pytest", "tests/test_gpu_gemm.py", "-q", "-x", "-k", sel],
                       cwd=root, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]


@pytest.mark.parametrize("pair,bn", [(0, 16), (0, 80), (0, 144), (0, 208), (0, 256), (1, 32), (1, 96), (1, 160), (1, 224)])
def test_token_tile_widths(torch_mod, pair, bn):
    """The token tile is chosen per call (tiles that fill whole waves of the persistent grid); TM_GEMM_BN pins it, at
    first use, so that every class of width (multiples of 32 and 16-column remainders, one and many token tiles) meets
    the full-check shapes - on the kernel with one SM per tile (TM_GEMM_PAIR=0) and on the CTA-pair kernel, which is
    the default wherever there are 256 weight rows."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, TM_GEMM_BN=str(bn), TM_GEMM_PAIR=str(pair))
    r = subprocess.run([sys.executable, "-m", "pytest", "tests/test_gpu_gemm.py", "-q", "-x", "-k", "test_small_shapes_full_check"],
                       cwd=root, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
