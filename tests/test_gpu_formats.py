"""The formats a GGUF-native container brings besides the five configured ones: GGUF's own Q4_0 (container dtype 9,
split nibbles), plain fp16 and bf16 rows (dtypes 3 and 10), and the path from a GGUF file to the decode lane.

Bars as everywhere on the path: dequantized weights bit-exact against the CPU oracle (for dtype 9 also against the
container Q4_0 the converter's nibble reorder makes of the same blocks), dots within 1e-3 * sum|w x| of the fp64 dot."""
from __future__ import annotations

import ctypes as C
import struct

import numpy as np
import pytest

from tensormark_b200 import chain, lib, synth
from tests.bounds import activation_rounding_bound
from tests.gpu_util import dev_bytes, dev_f32, gemv_dev, ptr, stream_ptr
from tests.test_gpu_dequant_gemv import same_bits
from tests.test_host_contracts import _gguf_bytes

pytestmark = pytest.mark.gpu
G9 = synth.GGUF_Q4_0


def _dequant(cuda, torch, dt, W, n, k):
    Wd = dev_bytes(torch, W)
    out = torch.empty(n * k, dtype=torch.float32, device="cuda")
    lib.check(cuda.tm_cuda_dequant_dev(ptr(Wd), ptr(out), n, k, dt, stream_ptr(torch)), "dequant")
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_gguf_q4_0_dequant_gemv_and_reorder(cuda, torch_mod, orc, golden):
    torch = torch_mod
    # the golden Q4_0 blocks (special scales included) read as split-nibble blocks
    blocks = golden["Q4_0_blocks"]
    got = _dequant(cuda, torch, G9, blocks, blocks.shape[0], 32)
    assert same_bits(got, orc.dequant(G9, blocks, blocks.shape[0] * 32))
    assert same_bits(got, orc.dequant(synth.Q4_0, orc.q4_split_to_interleaved(blocks), blocks.shape[0] * 32))
    for n, k in [(2048, 2048), (301, 2048), (64, 5632), (5, 96), (1187, 4096)]:
        W = synth.make_weights(G9, n, k, seed=60 + n)
        x = synth.make_activations(k, seed=61)
        assert np.array_equal(_dequant(cuda, torch, G9, W, n, k).view(np.uint32), orc.dequant(G9, W, n * k).view(np.uint32))
        Wd = dev_bytes(torch, W)
        y = gemv_dev(cuda, torch, G9, Wd, dev_f32(torch, x), n, k)
        y64, yabs = orc.gemv_f64(G9, W, x, n, k)
        err = np.abs(y - y64)
        assert np.all(err <= 1e-3 * yabs) and np.all(err <= activation_rounding_bound(orc, G9, W, x, n, k) + 2e-6 * yabs), (n, k)
        # the device reorder turns the same buffer into container Q4_0: identical weights, and the Q4_0 kernel agrees
        lib.check(cuda.tm_cuda_q4_0_from_gguf_dev(ptr(Wd), n * (k // 32), stream_ptr(torch)), "reorder")
        torch.cuda.synchronize()
        assert np.array_equal(Wd[: W.size].cpu().numpy(), orc.q4_split_to_interleaved(W).reshape(-1))
        y1 = gemv_dev(cuda, torch, synth.Q4_0, Wd, dev_f32(torch, x), n, k)
        assert np.all(np.abs(y1 - y64) <= 1e-3 * yabs)
    # prefill GEMM on the split-nibble blocks (operands dequantized by the generic pre-pass)
    m, n, k = 70, 192, 512
    W = synth.make_weights(G9, n, k, seed=70)
    A = synth.make_activations((m, k), seed=71)
    Cm = np.empty((m, n), np.float32)
    lib.check(cuda.tm_cuda_sgemm_q(A.ctypes.data, W.ctypes.data, Cm.ctypes.data, m, n, k, G9), "sgemm_q")
    ref = A.astype(np.float64) @ orc.dequant(G9, W, n * k).reshape(n, k).astype(np.float64).T
    absum = np.abs(A).astype(np.float64) @ np.abs(orc.dequant(G9, W, n * k).reshape(n, k)).astype(np.float64).T
    assert np.all(np.abs(Cm - ref) <= 1e-3 * absum)


@pytest.mark.parametrize("bf16", [False, True], ids=["fp16", "bf16"])
def test_plain_16bit_rows_gemv(cuda, torch_mod, bf16):
    torch = torch_mod
    rng = np.random.default_rng(80 + bf16)
    dt = synth.BF16 if bf16 else synth.F16
    for n, k in [(4096, 4096), (333, 2048), (7, 14336), (64, 100), (9, 31)]:       # the last two take the scalar-load kernel
        wf = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
        if bf16:
            bits = (wf.view(np.uint32) >> 16).astype(np.uint16)                    # truncation is fine: any bf16 pattern is a valid weight
            w = (bits.astype(np.uint32) << 16).view(np.float32)
        else:
            bits = wf.astype(np.float16).view(np.uint16)
            w = bits.view(np.float16).astype(np.float32)
        x = synth.make_activations(k, seed=81)
        Wd = dev_bytes(torch, bits.view(np.uint8))
        y = gemv_dev(cuda, torch, dt, Wd, dev_f32(torch, x), n, k)
        p = w.astype(np.float64) * x.astype(np.float64)[None, :]
        assert np.all(np.abs(y - p.sum(1)) <= 1e-3 * np.abs(p).sum(1)), (n, k)
        assert float((np.abs(y - p.sum(1)) / np.abs(p).sum(1)).max()) < 1e-5      # fp32 accumulation of exact products


def test_lane_f16_entries(cuda):
    """tok_gemv_h / tok_embed_h (metal_shim.mm:105-124): an F16 tensor registered with the lane, addressed by byte offset."""
    L = cuda
    XS, YS, TK = 70, 71, 72
    n, k = 96, 1024
    rng = np.random.default_rng(90)
    w16 = (rng.standard_normal((n, k)) * 0.05).astype(np.float16)
    pad = np.zeros(8, np.float16)
    blob = np.concatenate([pad, w16.reshape(-1)])                                   # the tensor starts 16 bytes into the handle
    x = synth.make_activations(k, seed=91)
    woff = C.c_uint64(0)
    wid = L.tm_cuda_tok_wbuf(blob.ctypes.data, blob.nbytes, None, 0, 0, C.byref(woff))
    assert wid >= 1000, lib.last_error()
    assert L.tm_cuda_tok_upload(XS, 0, x.ctypes.data, x.nbytes) and L.tm_cuda_tok_reserve(YS, 4 * n + 16)
    toks = np.array([5, 0xFFFFFFFF, 95], np.uint32)
    assert L.tm_cuda_tok_upload(TK, 0, toks.ctypes.data, toks.nbytes)
    assert L.tm_cuda_tok_begin()
    L.tm_cuda_tok_gemv_h(XS, wid, woff.value + 16, YS, 16, n, k)
    assert L.tm_cuda_tok_flush(), lib.last_error()
    y = np.empty(n, np.float32)
    assert L.tm_cuda_tok_download(YS, 16, y.ctypes.data, y.nbytes)
    p = w16.astype(np.float64) * x.astype(np.float64)[None, :]
    assert np.all(np.abs(y - p.sum(1)) <= 1e-3 * np.abs(p).sum(1))
    for idx, want in ((0, w16[5].astype(np.float32)), (1, np.zeros(k, np.float32)), (2, w16[95].astype(np.float32))):
        assert L.tm_cuda_tok_begin()
        L.tm_cuda_tok_embed_h(TK, idx, wid, woff.value + 16, XS, k)
        assert L.tm_cuda_tok_flush(), lib.last_error()
        row = np.empty(k, np.float32)
        assert L.tm_cuda_tok_download(XS, 0, row.ctypes.data, row.nbytes)
        assert np.array_equal(row, want)                                            # half -> float is exact; the sentinel gives zeros
    # out-of-range requests latch instead of launching
    assert L.tm_cuda_tok_begin()
    L.tm_cuda_tok_gemv_h(XS, wid, woff.value + 16, YS, 16, n + 1, k)
    assert not L.tm_cuda_tok_flush()


def test_gguf_file_to_lane(cuda, orc, tmp_path):
    """A GGUF file with split-nibble Q4_0 and Q6_K tensors: index -> one weight handle with aligned offsets -> the
    Q4_0 tensors reordered on the device -> lane GEMVs, against the oracle's reading of the file's own bytes."""
    L = cuda
    XS, YS = 73, 74
    n, k = 160, 2048
    wq = synth.make_weights(G9, n, k, seed=95)
    wh = synth.make_weights(synth.Q6_K, 48, k, seed=96)
    data = _gguf_bytes([("blk.0.attn_q.weight", 2, (k, n), wq.tobytes()), ("output.weight", 14, (k, 48), wh.tobytes())])
    path = tmp_path / "model.gguf"
    path.write_bytes(data)
    names = ["model.layers.0.self_attn.q_proj.weight", "lm_head.weight"]
    wid, info = chain.tmq_upload(str(path), names)
    assert info[names[0]][1] == synth.Q4_0 and info[names[0]][2] == n * (k // 32)      # dtype ON THE DEVICE: reordered
    assert info[names[1]][1] == synth.Q6_K
    x = synth.make_activations(k, seed=97)
    assert L.tm_cuda_tok_upload(XS, 0, x.ctypes.data, x.nbytes) and L.tm_cuda_tok_reserve(YS, 4 * n)
    for name, W, dt_file, rows in ((names[0], wq, G9, n), (names[1], wh, synth.Q6_K, 48)):
        woff, dt_dev, _ = info[name]
        assert L.tm_cuda_tok_begin()
        L.tm_cuda_tok_gemv_kq(XS, wid, woff, YS, 0, rows, k, dt_dev)
        assert L.tm_cuda_tok_flush(), lib.last_error()
        y = np.empty(rows, np.float32)
        assert L.tm_cuda_tok_download(YS, 0, y.ctypes.data, y.nbytes)
        y64, yabs = orc.gemv_f64(dt_file, W, x, rows, k)
        assert np.all(np.abs(y - y64) <= 1e-3 * yabs), name


def test_tq2_ternary_rows(cuda, torch_mod, orc, golden):
    """Container dtype 7 (tensormark/quant.h:446-566): dequant bit-exact (golden vectors from the reference's own build,
    its quantizer's output included), GEMV by the code-counting dot within the path's bar."""
    torch = torch_mod
    q = golden["TQ2_quantized_blocks"].reshape(-1, 34)
    got = _dequant(cuda, torch, synth.TQ2, q, q.shape[0], 128)
    assert np.array_equal(got.view(np.uint32), golden["TQ2_quantized_dequant_bits"])
    for n, k in [(512, 2048), (33, 4096), (3, 128)]:
        W = synth.make_weights(synth.TQ2, n, k, seed=40 + n)
        x = synth.make_activations(k, seed=41)
        assert np.array_equal(_dequant(cuda, torch, synth.TQ2, W, n, k).view(np.uint32), orc.dequant(synth.TQ2, W, n * k).view(np.uint32))
        y = gemv_dev(cuda, torch, synth.TQ2, dev_bytes(torch, W), dev_f32(torch, x), n, k)
        y64, yabs = orc.gemv_f64(synth.TQ2, W, x, n, k)
        assert np.all(np.abs(y - y64) <= 1e-3 * yabs), (n, k)
