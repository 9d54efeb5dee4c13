"""CPU: the restated oracle against the reference's golden vectors and own code."""
from __future__ import annotations

import numpy as np
import pytest

from oracle import binding
from tensormark_b200 import synth

DTYPES = [synth.Q8_0, synth.Q4_0, synth.Q4_1, synth.Q5_K, synth.Q6_K, synth.Q4_K, synth.TQ2]


@pytest.mark.parametrize("dt", DTYPES)
def test_dequant_matches_golden(orc, golden, dt):
    name = synth.DTYPE_NAMES[dt]
    blocks = golden[f"{name}_blocks"]
    want = golden[f"{name}_dequant_bits"]
    got = orc.dequant(dt, blocks, blocks.shape[0] * synth.BLOCK_ELEMS[dt]).view(np.uint32)
    # bit-exact, NaN payloads included
    assert np.array_equal(got, want)


@pytest.mark.parametrize("dt", [synth.Q8_0, synth.Q4_0, synth.TQ2])
def test_dequant_of_reference_quantized_rows(orc, golden, dt):
    name = synth.DTYPE_NAMES[dt]
    q = golden[f"{name}_quantized_blocks"]
    want = golden[f"{name}_quantized_dequant_bits"]
    got = orc.dequant(dt, q, want.size).view(np.uint32)
    assert np.array_equal(got, want)
    # round trip stays inside half a quantization step of the source (sanity on the fixture itself)
    x = golden[f"{name}_quantized_from"]
    be = synth.BLOCK_ELEMS[dt]
    # ternary: d = max|x| and codes -1, 0, +1, so a value can be off by half of d (plus the fp16 rounding of d)
    step = np.abs(x).reshape(-1, be).max(axis=1) / {synth.Q8_0: 127.0, synth.Q4_0: 8.0, synth.TQ2: 2.0}[dt]
    err = np.abs(got.view(np.float32) - x).reshape(-1, be).max(axis=1)
    assert np.all(err <= step * 1.01 + 1e-12)


def test_fp16_conversions_match_golden(orc, golden):
    want = golden["fp16_to_fp32_bits"]
    got = np.array([np.float32(orc.fp16_to_fp32(h)).view(np.uint32) for h in range(65536)], dtype=np.uint32)
    nan = (want & 0x7fffffff) > 0x7f800000
    assert np.array_equal(got[~nan], want[~nan])
    assert np.all((got[nan] & 0x7fffffff) > 0x7f800000)     # ctypes may quiet a signalling NaN in transit
    fin = golden["fp32_to_fp16_in_bits"].view(np.float32)
    hout = golden["fp32_to_fp16_out"]
    got16 = np.array([orc.fp32_to_fp16(float(v)) for v in fin], dtype=np.uint16)
    assert np.array_equal(got16, hout)


@pytest.mark.parametrize("dt", DTYPES)
def test_oracle_equals_reference_build_when_present(orc, dt):
    ref = binding.reference()
    if ref is None:
        pytest.skip("oracle/_ref was not built in this checkout (reference tree absent)")
    k = 1024
    W = synth.make_weights(dt, 32, k, seed=500 + dt)
    assert np.array_equal(orc.dequant(dt, W, 32 * k).view(np.uint32), ref.dequant(dt, W, 32 * k).view(np.uint32))


@pytest.mark.parametrize("dt", DTYPES)
def test_gemv_restatement_agrees_with_fp64(orc, dt):
    n, k = 48, 1024
    W = synth.make_weights(dt, n, k, seed=21)
    x = synth.make_activations(k, seed=22)
    y = orc.gemv(dt, W, x, n, k)
    y64, yabs = orc.gemv_f64(dt, W, x, n, k)
    assert np.all(np.abs(y - y64) <= 1e-5 * yabs)
    # the pool split must not change a single bit: rows are independent
    assert np.array_equal(orc.gemv(dt, W, x, n, k, threads=3).view(np.uint32), y.view(np.uint32))


def test_gemv_linearity_property(orc):
    # y(W, a*x1 + x2) == a*y(W, x1) + y(W, x2) up to rounding: a size-independent check of the dot path
    n, k = 16, 2048
    W = synth.make_weights(synth.Q4_0, n, k, seed=0)
    x1, x2 = synth.make_activations(k, 1), synth.make_activations(k, 2, stream=5)
    y = orc.gemv_f64(synth.Q4_0, W, (2.0 * x1 + x2).astype(np.float32), n, k)[0]
    y1 = orc.gemv_f64(synth.Q4_0, W, x1, n, k)[0]
    y2, ya = orc.gemv_f64(synth.Q4_0, W, x2, n, k)
    assert np.all(np.abs(y - (2 * y1 + y2)) <= 1e-5 * (ya + 1))


def test_gemm_restatement(orc):
    m, n, k = 5, 24, 512
    for dt in (synth.Q4_0, synth.Q6_K):
        W = synth.make_weights(dt, n, k, seed=4)
        A = synth.make_activations((m, k), seed=4)
        C = orc.gemm(dt, W, A, m, n, k, threads=2)
        for i in range(m):
            y64, yabs = orc.gemv_f64(dt, W, A[i], n, k)
            assert np.all(np.abs(C[i] - y64) <= 1e-5 * yabs)


def test_bad_arguments_are_rejected(orc):
    W = synth.make_weights(synth.Q4_0, 2, 64, seed=1)
    with pytest.raises(ValueError):
        orc.gemv(synth.Q4_0, W, np.zeros(48, np.float32), 2, 48)      # K not a multiple of 32
    with pytest.raises(ValueError):
        orc.dequant(synth.Q6_K, W, 128)                              # not whole super-blocks


def test_glue_restatements(orc):
    rng = np.random.default_rng(3)
    x = rng.standard_normal(256).astype(np.float32)
    w = rng.standard_normal(256).astype(np.float32)
    got = orc.rmsnorm(x, w, 1e-5)
    want = x / np.sqrt(np.mean(x.astype(np.float64) ** 2) + 1e-5) * w
    assert np.allclose(got, want, rtol=1e-5, atol=1e-6)
    # rope: a rotation preserves the norm of every (j, j + dh/2) pair and position 0 is the identity
    r = rng.standard_normal(128).astype(np.float32)
    assert np.array_equal(orc.rope_head(r, 0, 5e5), r)
    rr = orc.rope_head(r, 77, 5e5)
    assert np.allclose(r[:64] ** 2 + r[64:] ** 2, rr[:64] ** 2 + rr[64:] ** 2, rtol=1e-5)
    tbl = orc.rope_table(128, 80, 5e5)
    a, b = r[:64], r[64:]
    assert np.allclose(rr[:64], a * tbl[77, :, 0] - b * tbl[77, :, 1], rtol=1e-6, atol=1e-7)
    # attention against a float64 softmax
    q = rng.standard_normal((4, 64)).astype(np.float32)
    K = rng.standard_normal((37, 64)).astype(np.float32)
    V = rng.standard_normal((37, 64)).astype(np.float32)
    got = orc.attn_group(q, K, V, 0.125)
    s = (q.astype(np.float64) @ K.T.astype(np.float64)) * 0.125
    p = np.exp(s - s.max(axis=1, keepdims=True)); p /= p.sum(axis=1, keepdims=True)
    assert np.allclose(got, p @ V, rtol=1e-4, atol=1e-5)
    g = rng.standard_normal(64).astype(np.float32); u = rng.standard_normal(64).astype(np.float32)
    assert np.allclose(orc.silu_mul(g, u), g / (1 + np.exp(-g.astype(np.float64))) * u, rtol=1e-5, atol=1e-6)
    assert orc.argmax(np.array([1, 5, 5, 2], np.float32)) == 1      # ties -> lowest index


def test_gguf_q4_0_equals_repacked_q4_0(orc):
    """Container dtype 9 (GGUF's split-nibble Q4_0, tensormark/llama.h:4588-4597) holds the same weights as the block the
    converter's nibble reorder makes of it (tensormark/convert_gguf.cpp:124-135): two independent statements of the
    layout, one checked against the other bit for bit, on random blocks and on the golden special-scale blocks."""
    import numpy as np
    from tensormark_b200 import synth
    W = synth.make_weights(synth.GGUF_Q4_0, 64, 2048, seed=9)
    a = orc.dequant(synth.GGUF_Q4_0, W, 64 * 2048)
    b = orc.dequant(synth.Q4_0, orc.q4_split_to_interleaved(W), 64 * 2048)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    # and it is NOT the interleaved reading of the same bytes
    assert not np.array_equal(a, orc.dequant(synth.Q4_0, W, 64 * 2048))
    # element j comes from the low nibble of byte j, element j + 16 from its high nibble
    blk = np.zeros(18, np.uint8); blk[0:2] = np.array([1.0], np.float16).view(np.uint8); blk[2] = 0x3C
    x = orc.dequant(synth.GGUF_Q4_0, blk, 32)
    assert x[0] == 0xC - 8 and x[16] == 0x3 - 8 and x[1] == -8
