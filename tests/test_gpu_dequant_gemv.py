"""GPU parity: dequantized weights bit-exact, dot products within 1e-3 * sum|w x| (fp32 accumulate).

Every call goes through the C ABI of libtm_cuda.so. The checker is the CPU oracle (and the
golden vectors produced by the reference's own quant.h)."""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

from tensormark_b200 import lib, synth
from tests.bounds import activation_rounding_bound
from tests.gpu_util import dev_bytes, dev_f32, gemv_dev, ptr, stream_ptr

pytestmark = pytest.mark.gpu
DTYPES = [synth.Q8_0, synth.Q4_0, synth.Q4_1, synth.Q5_K, synth.Q6_K, synth.Q4_K]
DEQUANT_DTYPES = DTYPES + [synth.TQ2]        # the ternary pack: bit-exact dequant and a plain (not streaming) GEMV
TOL = 1e-3      # relative to sum_k |w_k x_k| per output, the bar the path is judged by


def same_bits(got: np.ndarray, want: np.ndarray) -> bool:
    """Bit-for-bit equality; a NaN must be a NaN on both sides (its payload is the multiplier hardware's
    choice: x86 propagates the operand's payload, the GPU returns the canonical quiet NaN)."""
    g, w = got.view(np.uint32), want.view(np.uint32)
    gn, wn = (g & 0x7fffffff) > 0x7f800000, (w & 0x7fffffff) > 0x7f800000
    return bool(np.array_equal(gn, wn) and np.array_equal(g[~gn], w[~wn]))


def _dequant_dev(cuda, torch, dt, blocks, n, k):
    W = dev_bytes(torch, blocks)
    out = torch.empty(n * k, dtype=torch.float32, device="cuda")
    lib.check(cuda.tm_cuda_dequant_dev(ptr(W), ptr(out), n, k, dt, stream_ptr(torch)), "tm_cuda_dequant_dev")
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("dt", DEQUANT_DTYPES)
def test_dequant_bit_exact_vs_golden(cuda, torch_mod, golden, dt):
    name = synth.DTYPE_NAMES[dt]
    blocks = golden[f"{name}_blocks"]
    be = synth.BLOCK_ELEMS[dt]
    # present the blocks as rows of one block each so special-scale blocks are covered too
    got = _dequant_dev(cuda, torch_mod, dt, blocks, blocks.shape[0], be)
    want = golden[f"{name}_dequant_bits"]
    assert same_bits(got, want)
    assert ((want & 0x7fffffff) > 0x7f800000).sum() > 0          # the fixture really holds NaN scales


@pytest.mark.parametrize("dt", DTYPES)
def test_dequant_bit_exact_vs_oracle_config_shapes(cuda, torch_mod, orc, dt):
    shapes = [(96, 2048), (40, 5632)] if dt in (synth.Q8_0, synth.Q4_0, synth.Q4_1) else [(64, 4096), (24, 14336)]
    for n, k in shapes:
        W = synth.make_weights(dt, n, k, seed=3)
        got = _dequant_dev(cuda, torch_mod, dt, W, n, k)
        assert np.array_equal(got.view(np.uint32), orc.dequant(dt, W, n * k).view(np.uint32))


def test_dequant_host_pointer_entry(cuda, orc):
    n, k = 33, 1024
    W = synth.make_weights(synth.Q6_K, n, k, seed=6)
    out = np.empty(n * k, np.float32)
    lib.check(cuda.tm_cuda_dequant(W.ctypes.data, out.ctypes.data, n, k, synth.Q6_K), "tm_cuda_dequant")
    assert np.array_equal(out.view(np.uint32), orc.dequant(synth.Q6_K, W, n * k).view(np.uint32))


def _check_gemv(cuda, torch, orc, dt, n, k, seed, wseed=None):
    W = synth.make_weights(dt, n, k, seed=seed if wseed is None else wseed)
    x = synth.make_activations(k, seed=seed)
    y = gemv_dev(cuda, torch, dt, dev_bytes(torch, W), dev_f32(torch, x), n, k)
    y64, yabs = orc.gemv_f64(dt, W, x, n, k)
    err = np.abs(y - y64)
    assert np.all(err <= TOL * yabs), (synth.DTYPE_NAMES[dt], n, k, float((err / yabs).max()))
    # ... and inside what the kernel's activation format can lose (tests/bounds.py) plus fp32 accumulation noise
    assert np.all(err <= activation_rounding_bound(orc, dt, W, x, n, k) + 2e-6 * yabs), (synth.DTYPE_NAMES[dt], n, k)
    return float((err / np.maximum(yabs, 1e-30)).max())


def test_config1_q4_0_2048(cuda, torch_mod, orc):
    worst = _check_gemv(cuda, torch_mod, orc, synth.Q4_0, 2048, 2048, seed=0)
    assert worst < 2e-5          # two-digit activations: derived worst case 9e-5 for one-scale inputs, a few 1e-6 in practice


@pytest.mark.parametrize("dt,seed", [(synth.Q8_0, 1), (synth.Q4_1, 2)])
@pytest.mark.parametrize("shape", synth.TINYLLAMA_SHAPES)
def test_config2_tinyllama_sweep(cuda, torch_mod, orc, dt, seed, shape):
    _check_gemv(cuda, torch_mod, orc, dt, shape[0], shape[1], seed=seed)


@pytest.mark.parametrize("dt", [synth.Q5_K, synth.Q6_K, synth.Q4_K])
@pytest.mark.parametrize("shape", synth.LLAMA3_8B_SHAPES)
def test_config3_kquant_llama3_shapes(cuda, torch_mod, orc, dt, shape):
    _check_gemv(cuda, torch_mod, orc, dt, shape[0], shape[1], seed=3)


@pytest.mark.parametrize("dt", DTYPES)
def test_ragged_and_minimum_shapes(cuda, torch_mod, orc, dt):
    be = synth.BLOCK_ELEMS[dt]
    # one row, rows not a multiple of the warp row group, a single block per row, an odd block count,
    # rows whose byte length is not a multiple of 16 (takes the byte-granular kernel)
    for n, k in [(1, 2048), (7, 4096), (3, be), (5, 3 * be), (301, 2048), (2, 11 * be), (1187, 2048)]:
        _check_gemv(cuda, torch_mod, orc, dt, n, k, seed=40 + n)


@pytest.mark.parametrize("dt", DTYPES)
def test_unaligned_weight_base_uses_generic_kernel(cuda, torch_mod, orc, dt):
    n, k = 19, 2048
    W = synth.make_weights(dt, n, k, seed=9)
    x = synth.make_activations(k, seed=9)
    buf = torch_mod.zeros(W.size + 64, dtype=torch_mod.uint8, device="cuda")
    buf[6: 6 + W.size] = torch_mod.from_numpy(W.reshape(-1)).cuda()
    view = buf[6:]
    y = gemv_dev(cuda, torch_mod, dt, view, dev_f32(torch_mod, x), n, k)
    y64, yabs = orc.gemv_f64(dt, W, x, n, k)
    assert np.all(np.abs(y - y64) <= TOL * yabs)


@pytest.mark.parametrize("dt", DTYPES)
def test_segmented_is_bit_identical_to_separate(cuda, torch_mod, dt):
    """q|k|v in one launch: every row must come out exactly as from its own launch (tensormark/metal.h:504-510)."""
    torch = torch_mod
    k = 2048 if dt in (synth.Q8_0, synth.Q4_0, synth.Q4_1) else 4096
    rows = [256, 64, 62]
    parts = [synth.make_weights(dt, r, k, seed=60 + i) for i, r in enumerate(rows)]
    x = dev_f32(torch, synth.make_activations(k, seed=61))
    # lay the tensors out with gaps, 16-byte aligned, as they would sit in a mapped file
    offs, cur = [], 48
    for p in parts:
        offs.append(cur)
        cur = (cur + p.size + 15) // 16 * 16 + 32
    blob = torch.zeros(cur + 64, dtype=torch.uint8, device="cuda")
    for p, o in zip(parts, offs):
        blob[o: o + p.size] = torch.from_numpy(p.reshape(-1)).cuda()
    n = sum(rows)
    y = torch.empty(n, dtype=torch.float32, device="cuda")
    woff = (C.c_uint64 * 3)(*offs)
    srows = (C.c_uint * 3)(*rows)
    lib.check(cuda.tm_cuda_gemv_seg_dev(ptr(x), ptr(blob), ptr(y), n, k, dt, woff, srows, 3, stream_ptr(torch)), "gemv_seg")
    torch.cuda.synchronize()
    got = y.cpu().numpy()
    start = 0
    for p, r in zip(parts, rows):
        sep = gemv_dev(cuda, torch, dt, dev_bytes(torch, p), x, r, k)
        assert np.array_equal(sep.view(np.uint32), got[start: start + r].view(np.uint32))
        start += r


def test_host_pointer_gemv_and_errors(cuda, orc):
    n, k = 512, 2048
    W = synth.make_weights(synth.Q4_0, n, k, seed=0)
    x = synth.make_activations(k, seed=0)
    y = np.empty(n, np.float32)
    lib.check(cuda.tm_cuda_q4_gemv(x.ctypes.data, W.ctypes.data, y.ctypes.data, n, k), "tm_cuda_q4_gemv")
    y64, yabs = orc.gemv_f64(synth.Q4_0, W, x, n, k)
    assert np.all(np.abs(y - y64) <= TOL * yabs)
    # second call hits the cached device copy and must give the same bits
    y2 = np.empty(n, np.float32)
    assert cuda.tm_cuda_q4_gemv(x.ctypes.data, W.ctypes.data, y2.ctypes.data, n, k)
    assert np.array_equal(y.view(np.uint32), y2.view(np.uint32))
    # the reference returns false for K % 32 != 0 (metal.h:2062) and the fallback counter moves
    before = cuda.tm_cuda_fallback_count()
    assert not cuda.tm_cuda_q4_gemv(x.ctypes.data, W.ctypes.data, y.ctypes.data, n, 2040)
    assert not cuda.tm_cuda_gemv_q(x.ctypes.data, W.ctypes.data, y.ctypes.data, n, 2048 + 32, synth.Q6_K)
    assert not cuda.tm_cuda_q4_gemv(None, W.ctypes.data, y.ctypes.data, n, k)
    assert cuda.tm_cuda_fallback_count() == before + 3
    assert lib.last_error() != ""
    cuda.tm_cuda_release_weights()


def test_empty_output_is_a_no_op(cuda, torch_mod):
    x = dev_f32(torch_mod, np.zeros(2048, np.float32))
    W = dev_bytes(torch_mod, np.zeros(16, np.uint8))
    y = torch_mod.empty(1, dtype=torch_mod.float32, device="cuda")
    assert cuda.tm_cuda_gemv_q_dev(ptr(x), ptr(W), ptr(y), 0, 2048, synth.Q4_0, stream_ptr(torch_mod))


def test_full_size_property_scaling_and_linearity(cuda, torch_mod, orc):
    """At the largest configured sizes the oracle is not rerun on every row; instead a size-independent property:
    W(a*x1 + x2) == a*W(x1) + W(x2) within rounding, for every output row. Each of the three results may be off
    by its own rounding, a small fraction of sum|w x| (the contract is 1e-3 of it); sum|w x| itself comes from the
    oracle on a sample of rows and, as rows of one random tensor have similar norms, bounds the others with slack."""
    torch = torch_mod
    for dt, (n, k) in [(synth.Q8_0, (32000, 2048)), (synth.Q6_K, (14336, 4096)), (synth.Q5_K, (4096, 14336))]:
        Wh = synth.make_weights(dt, n, k, seed=5)
        W = dev_bytes(torch, Wh)
        x1 = synth.make_activations(k, seed=5)
        x2 = synth.make_activations(k, seed=6)
        x3 = (2.0 * x1 + x2).astype(np.float32)
        y1 = gemv_dev(cuda, torch, dt, W, dev_f32(torch, x1), n, k).astype(np.float64)
        y2 = gemv_dev(cuda, torch, dt, W, dev_f32(torch, x2), n, k).astype(np.float64)
        y = gemv_dev(cuda, torch, dt, W, dev_f32(torch, x3), n, k).astype(np.float64)
        rows = np.unique(np.random.default_rng(0).integers(0, n, size=128))
        sub = np.ascontiguousarray(Wh[rows])
        yabs = sum(c * orc.gemv_f64(dt, sub, x, rows.size, k)[1] for c, x in ((2.0, x1), (1.0, x2), (1.0, x3)))
        dev = np.abs(y - (2 * y1 + y2))
        assert np.all(dev[rows] <= 1e-4 * yabs)                     # sampled rows against their own sum|w x|
        assert np.all(dev <= 2e-4 * float(yabs.max()))              # every row against the sample's largest
