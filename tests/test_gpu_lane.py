"""GPU parity of the token lane (slots, weight handles, decode glue, attention, argmax) against the CPU oracle.

The calls follow the order the reference's token encoder makes them (tensormark/llama.h:5818-5924);
fp32 glue is compared at 1e-3 relative (the reference's GPU-vs-CPU bar, test_llama_gpu_stack.cpp:10-14)
or tighter where the arithmetic is exact."""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

from tensormark_b200 import lib, synth
from tests.gpu_util import dev_f32, ptr, stream_ptr

pytestmark = pytest.mark.gpu

# slot ids, as the reference engine numbers its own (llama.h:1245-1250 style)
X, H_, QKV, AO, TOK, LOGITS, PROBS, KC, VC, T0, T1, BIAS = range(12)


def up(cuda, slot, arr, off=0):
    a = np.ascontiguousarray(arr)
    lib.check(cuda.tm_cuda_tok_upload(slot, off, a.ctypes.data, a.nbytes), "tok_upload")


def down(cuda, slot, n, dtype=np.float32, off=0):
    out = np.empty(n, dtype=dtype)
    lib.check(cuda.tm_cuda_tok_download(slot, off, out.ctypes.data, out.nbytes), "tok_download")
    return out


_KEEP = []      # registrations are keyed by host address: keep every registered array alive for the whole run


def wbuf(cuda, W):
    _KEEP.append(W)
    woff = C.c_uint64(0)
    wid = cuda.tm_cuda_tok_wbuf(W.ctypes.data, W.nbytes, None, 0, 0, C.byref(woff))
    assert wid >= 1000, lib.last_error()
    return wid, woff.value


def test_slots_upload_download_and_growth_rule(cuda):
    a = np.arange(100, dtype=np.float32)
    up(cuda, T0, a)
    assert np.array_equal(down(cuda, T0, 100), a)
    assert np.array_equal(down(cuda, T0, 10, off=40), a[10:20])
    # a slot may be created but not grown while a token is being encoded (metal.h:2268-2270)
    assert cuda.tm_cuda_tok_begin()
    assert not cuda.tm_cuda_tok_reserve(T0, 1 << 20)
    cuda.tm_cuda_tok_add(T0, T0, 100000)           # needs more than the slot holds: latches, launches nothing
    assert not cuda.tm_cuda_tok_end(T0, None, 0)
    assert "reserved before token encoding" in lib.last_error()
    # the lane is usable again afterwards and the data is untouched
    assert cuda.tm_cuda_tok_begin() and cuda.tm_cuda_tok_end(T0, None, 0)
    assert np.array_equal(down(cuda, T0, 100), a)
    assert cuda.tm_cuda_tok_reserve(T0, 1 << 20)    # growing between tokens keeps the contents
    assert np.array_equal(down(cuda, T0, 100), a)


@pytest.mark.parametrize("dt", [synth.Q4_0, synth.Q8_0, synth.Q4_1, synth.Q5_K, synth.Q6_K])
def test_tok_gemv_all_dtypes(cuda, orc, dt):
    n, k = 320, 2048
    W = synth.make_weights(dt, n, k, seed=90 + dt)
    x = synth.make_activations(k, seed=91)
    wid, woff = wbuf(cuda, W)
    # registering the same tensor again returns the same handle (metal.h:3305-3310)
    assert wbuf(cuda, W) == (wid, woff)
    up(cuda, X, x)
    assert cuda.tm_cuda_tok_reserve(T1, 4 * (n + 8))
    assert cuda.tm_cuda_tok_begin()
    if dt == synth.Q4_0:
        cuda.tm_cuda_tok_gemv(X, wid, woff, T1, 32, n, k)           # byte offset 32 into the output slot
    else:
        cuda.tm_cuda_tok_gemv_kq(X, wid, woff, T1, 32, n, k, dt)
    y = np.empty(n, np.float32)
    assert cuda.tm_cuda_tok_end(T1, None, 0), lib.last_error()
    y = down(cuda, T1, n, off=32)
    y64, yabs = orc.gemv_f64(dt, W, x, n, k)
    assert np.all(np.abs(y - y64) <= 1e-3 * yabs)


def test_zero_copy_mapping_and_segmented_qkv(cuda, orc):
    """Three tensors inside one "mapped file": one handle, byte offsets, one fused q|k|v launch
    (llama.h:5871-5881) that equals the three separate ones bit for bit."""
    k, rows = 2048, [512, 128, 128]
    parts = [synth.make_weights(synth.Q4_0, r, k, seed=100 + i) for i, r in enumerate(rows)]
    blob = np.zeros(sum(p.size for p in parts) + 4096, dtype=np.uint8)
    offs, cur = [], 160
    for p in parts:
        offs.append(cur)
        blob[cur: cur + p.size] = p.reshape(-1)
        cur += (p.size + 15) // 16 * 16 + 16
    _KEEP.append(blob)
    ids = []
    for p, o in zip(parts, offs):
        woff = C.c_uint64(0)
        wid = cuda.tm_cuda_tok_wbuf(blob.ctypes.data + o, p.size, blob.ctypes.data, blob.nbytes, 1, C.byref(woff))
        assert wid >= 1000 and woff.value == o
        ids.append(wid)
    assert len(set(ids)) == 1
    # outside the mapping -> refused
    woff = C.c_uint64(0)
    assert cuda.tm_cuda_tok_wbuf(blob.ctypes.data + blob.nbytes + 64, 16, blob.ctypes.data, blob.nbytes, 1, C.byref(woff)) == -1
    x = synth.make_activations(k, seed=101)
    up(cuda, X, x)
    n = sum(rows)
    assert cuda.tm_cuda_tok_reserve(QKV, 4 * n) and cuda.tm_cuda_tok_reserve(T1, 4 * n)
    assert cuda.tm_cuda_tok_gemv_seg_supported(synth.Q4_0) and not cuda.tm_cuda_tok_gemv_seg_supported(synth.F16)
    assert cuda.tm_cuda_tok_begin()
    cuda.tm_cuda_tok_gemv_seg(X, ids[0], QKV, 0, n, k, (C.c_uint64 * 3)(*offs), (C.c_uint * 3)(*rows), 3)
    yo = 0
    for r, o in zip(rows, offs):
        cuda.tm_cuda_tok_gemv(X, ids[0], o, T1, 4 * yo, r, k)
        yo += r
    assert cuda.tm_cuda_tok_end(QKV, None, 0), lib.last_error()
    fused, sep = down(cuda, QKV, n), down(cuda, T1, n)
    assert np.array_equal(fused.view(np.uint32), sep.view(np.uint32))
    ref = np.concatenate([orc.gemv_f64(synth.Q4_0, p, x, r, k)[0] for p, r in zip(parts, rows)])
    yabs = np.concatenate([orc.gemv_f64(synth.Q4_0, p, x, r, k)[1] for p, r in zip(parts, rows)])
    assert np.all(np.abs(fused - ref) <= 1e-3 * yabs)
    # a segment table whose rows do not add up is a caller error: sticky, nothing launched
    assert cuda.tm_cuda_tok_begin()
    cuda.tm_cuda_tok_gemv_seg(X, ids[0], QKV, 0, n + 1, k, (C.c_uint64 * 3)(*offs), (C.c_uint * 3)(*rows), 3)
    assert not cuda.tm_cuda_tok_end(QKV, None, 0)


def test_elementwise_glue(cuda, orc):
    rng = np.random.default_rng(5)
    d = 4096
    x = rng.standard_normal(d).astype(np.float32) * 3
    w = (1 + 0.02 * rng.standard_normal(d)).astype(np.float32)
    b = rng.standard_normal(d).astype(np.float32)
    _KEEP.append(w)
    up(cuda, X, x); up(cuda, T0, b)
    assert cuda.tm_cuda_tok_reserve(H_, 4 * d)
    assert cuda.tm_cuda_tok_begin()
    cuda.tm_cuda_tok_rmsnorm(X, w.ctypes.data, H_, d, 1e-5)
    cuda.tm_cuda_tok_add(X, T0, d)
    assert cuda.tm_cuda_tok_end(H_, None, 0), lib.last_error()
    assert np.allclose(down(cuda, H_, d), orc.rmsnorm(x, w, 1e-5), rtol=2e-6, atol=1e-7)
    assert np.array_equal(down(cuda, X, d), x + b)
    # silu(g) * u on the packed gate|up slot, byte offsets as the engine passes them (llama.h:5903)
    f = 1000
    gu = rng.standard_normal(2 * f).astype(np.float32) * 2
    up(cuda, T1, gu)
    assert cuda.tm_cuda_tok_begin()
    cuda.tm_cuda_tok_silu_mul(T1, 0, T1, 4 * f, f)
    assert cuda.tm_cuda_tok_end(T1, None, 0)
    assert np.allclose(down(cuda, T1, f), orc.silu_mul(gu[:f], gu[f:]), rtol=2e-6, atol=1e-7)
    # qkv bias
    up(cuda, BIAS, b[: 2 * f]); up(cuda, T1, gu)
    assert cuda.tm_cuda_tok_begin()
    cuda.tm_cuda_tok_bias_qkv(T1, BIAS, 4 * 100, 500)
    assert cuda.tm_cuda_tok_end(T1, None, 0)
    assert np.array_equal(down(cuda, T1, 500), gu[:500] + b[100:600])


@pytest.mark.parametrize("kv_half_env", ["half"])
def test_rope_kv_cache_and_attention(cuda, orc, kv_half_env):
    """Config-5 head geometry: 32 query heads, 8 KV heads of 128, positions up to 639, theta 5e5."""
    Hn, KVH, dh, ctx, theta = 32, 8, 128, 768, 500000.0
    QD, KVD, REP = Hn * dh, KVH * dh, Hn // KVH
    rng = np.random.default_rng(7)
    allow = 640
    # fill the caches through the lane: for each position rope(k) -> cache, v -> cache
    ks = rng.standard_normal((allow, KVD)).astype(np.float32)
    vs = rng.standard_normal((allow, KVD)).astype(np.float32)
    n_cache = KVH * ctx * dh
    assert cuda.tm_cuda_tok_kv_reserve(KC, n_cache) and cuda.tm_cuda_tok_kv_reserve(VC, n_cache)
    assert cuda.tm_cuda_tok_reserve(QKV, 4 * (QD + 2 * KVD)) and cuda.tm_cuda_tok_reserve(PROBS, 4 * Hn * ctx)
    assert cuda.tm_cuda_tok_reserve(AO, 4 * QD)
    # bulk rows [0, allow-8) arrive as an fp32 upload (the engine uploads its prefill rows, llama.h:5738-5744)
    kref = np.zeros((KVH, ctx, dh), np.float32); vref = np.zeros_like(kref)
    for p in range(allow):
        for h in range(KVH):
            kref[h, p] = orc.rope_head(ks[p, h * dh:(h + 1) * dh], p, theta)
            vref[h, p] = vs[p, h * dh:(h + 1) * dh]
    bulk = allow - 8
    for h in range(KVH):
        lib.check(cuda.tm_cuda_tok_kv_upload(KC, (h * ctx) * dh, np.ascontiguousarray(kref[h, :bulk]).ctypes.data, bulk * dh), "kv_upload")
        lib.check(cuda.tm_cuda_tok_kv_upload(VC, (h * ctx) * dh, np.ascontiguousarray(vref[h, :bulk]).ctypes.data, bulk * dh), "kv_upload")
    # the last 8 positions go through rope_k_cache / v_cache kernels
    for p in range(bulk, allow):
        qkv = np.concatenate([np.zeros(QD, np.float32), ks[p], vs[p]])
        up(cuda, QKV, qkv)
        assert cuda.tm_cuda_tok_begin()
        cuda.tm_cuda_tok_rope_k_cache(QKV, 4 * QD, KC, KVH, dh, ctx, p, theta)
        cuda.tm_cuda_tok_v_cache(QKV, 4 * (QD + KVD), VC, KVH, dh, ctx, p)
        assert cuda.tm_cuda_tok_end(QKV, None, 0), lib.last_error()
    # read a few rows back: half storage rounds once, so compare against the fp16-rounded reference
    back = np.empty(dh, np.float32)
    for (h, p) in [(0, 0), (3, bulk - 1), (7, allow - 1), (2, bulk)]:
        lib.check(cuda.tm_cuda_tok_kv_download(KC, (h * ctx + p) * dh, back.ctypes.data, dh), "kv_download")
        want = kref[h, p].astype(np.float16).astype(np.float32)
        assert np.allclose(back, want, rtol=1.1e-3, atol=1e-6), (h, p)
    # query: rope in place, then attention
    q = rng.standard_normal(QD).astype(np.float32)
    pos = allow - 1
    up(cuda, QKV, np.concatenate([q, ks[pos], vs[pos]]))
    assert cuda.tm_cuda_tok_begin()
    cuda.tm_cuda_tok_rope_q(QKV, Hn, dh, pos, theta)
    cuda.tm_cuda_tok_attn(QKV, KC, VC, PROBS, AO, QD, Hn, KVH, dh, ctx, allow, 1.0 / np.sqrt(dh), REP)
    assert cuda.tm_cuda_tok_end(AO, None, 0), lib.last_error()
    qr = down(cuda, QKV, QD)
    qref = np.concatenate([orc.rope_head(q[h * dh:(h + 1) * dh], pos, theta) for h in range(Hn)])
    assert np.allclose(qr, qref, rtol=1e-5, atol=1e-6)
    got = down(cuda, AO, QD).reshape(Hn, dh)
    kh = kref.astype(np.float16).astype(np.float32); vh = vref.astype(np.float16).astype(np.float32)
    for g in range(KVH):
        want = orc.attn_group(qref.reshape(Hn, dh)[g * REP:(g + 1) * REP], kh[g, :allow], vh[g, :allow], 1.0 / np.sqrt(dh))
        assert np.allclose(got[g * REP:(g + 1) * REP], want, rtol=1e-3, atol=2e-5), g
    # invalid geometry is refused like the reference's argument check (metal.h:4157-4160)
    assert cuda.tm_cuda_tok_begin()
    cuda.tm_cuda_tok_attn(QKV, KC, VC, PROBS, AO, QD, Hn, KVH, dh, ctx, ctx + 1, 0.1, REP)
    assert not cuda.tm_cuda_tok_end(AO, None, 0)


@pytest.mark.parametrize("allow", [1, 5, 130, 511])
@pytest.mark.parametrize("kv_half", [0, 1])
def test_attention_device_entry_short_and_ragged(cuda, torch_mod, orc, allow, kv_half):
    torch = torch_mod
    Hn, KVH, dh, ctx = 8, 2, 64, 512
    rng = np.random.default_rng(allow)
    q = rng.standard_normal((Hn, dh)).astype(np.float32)
    K = rng.standard_normal((KVH, ctx, dh)).astype(np.float32)
    V = rng.standard_normal((KVH, ctx, dh)).astype(np.float32)
    if kv_half:
        K = K.astype(np.float16).astype(np.float32); V = V.astype(np.float16).astype(np.float32)
    qd = dev_f32(torch, q)
    kd = torch.from_numpy(K).cuda(); vd = torch.from_numpy(V).cuda()
    if kv_half:
        kd, vd = kd.half(), vd.half()
    need = cuda.tm_cuda_attn_decode_scratch(Hn, KVH, dh, ctx, allow)
    sc = torch.empty(need // 4 + 1, dtype=torch.float32, device="cuda")
    out = torch.empty(Hn * dh, dtype=torch.float32, device="cuda")
    lib.check(cuda.tm_cuda_attn_decode_dev(ptr(qd), ptr(kd), ptr(vd), ptr(sc), need, ptr(out), Hn, KVH, dh, ctx, allow,
                                           0.125, kv_half, stream_ptr(torch)), "attn_decode_dev")
    torch.cuda.synchronize()
    got = out.cpu().numpy().reshape(Hn, dh)
    rep = Hn // KVH
    for g in range(KVH):
        want = orc.attn_group(q[g * rep:(g + 1) * rep], K[g, :allow], V[g, :allow], 0.125)
        assert np.allclose(got[g * rep:(g + 1) * rep], want, rtol=1e-3, atol=2e-5)


def test_argmax_sample_embed_and_chain_peek(cuda, orc):
    v, d = 128256, 2048
    rng = np.random.default_rng(11)
    logits = rng.standard_normal(v).astype(np.float32)
    logits[77] = logits[90001] = 9.5          # a tie: the lowest index wins (metal.h:2335)
    logits[5] = np.nan
    up(cuda, LOGITS, logits)
    sentinel = np.full(4, 0xFFFFFFFF, np.uint32)
    up(cuda, TOK, sentinel)
    assert cuda.tm_cuda_tok_peek(TOK, 0) == 0xFFFFFFFF
    E = synth.make_weights(synth.Q4_0, 300, d, seed=12)
    E6 = synth.make_weights(synth.Q6_K, 300, d, seed=13)
    wid, woff = wbuf(cuda, E)
    wid6, woff6 = wbuf(cuda, E6)
    assert cuda.tm_cuda_tok_reserve(X, 4 * d) and cuda.tm_cuda_tok_reserve(H_, 4 * d)
    assert cuda.tm_cuda_tok_begin()
    cuda.tm_cuda_tok_argmax(LOGITS, TOK, 0, v)
    cuda.tm_cuda_tok_embed_q4(TOK, 0, wid, woff, X, d)            # row of the token just chosen, on the device
    cuda.tm_cuda_tok_embed_kq(TOK, 0, wid6, woff6, H_, d, synth.Q6_K)
    cuda.tm_cuda_tok_embed_q4(TOK, 1, wid, woff, T0, d)           # entry 1 still holds the sentinel -> zeros
    assert cuda.tm_cuda_tok_end_async()
    assert cuda.tm_cuda_tok_wait_pending(), lib.last_error()
    assert cuda.tm_cuda_tok_peek(TOK, 0) == 77
    assert orc.argmax(np.nan_to_num(logits, nan=-np.inf)) == 77
    assert np.array_equal(down(cuda, X, d).view(np.uint32), orc.dequant(synth.Q4_0, E[77], d).view(np.uint32))
    assert np.array_equal(down(cuda, H_, d).view(np.uint32), orc.dequant(synth.Q6_K, E6[77], d).view(np.uint32))
    assert not down(cuda, T0, d).any()
    # repeated argmax re-arms its scratch: same answer every time, on a different index
    logits[123456] = 20.0
    up(cuda, LOGITS, logits)
    for i in (1, 2, 3):
        assert cuda.tm_cuda_tok_begin()
        cuda.tm_cuda_tok_argmax(LOGITS, TOK, i, v)
        assert cuda.tm_cuda_tok_end(TOK, None, 0)
    assert list(down(cuda, TOK, 4, np.uint32)) == [77, 123456, 123456, 123456]
    # Gumbel-max: deterministic per (seed, idx); a near-zero temperature reproduces the argmax
    picks = []
    for seed in (1, 1, 2):
        assert cuda.tm_cuda_tok_begin()
        cuda.tm_cuda_tok_sample(LOGITS, TOK, 0, v, 1.0, seed)
        assert cuda.tm_cuda_tok_end(TOK, None, 0)
        picks.append(int(down(cuda, TOK, 1, np.uint32)[0]))
    assert picks[0] == picks[1] and 0 <= picks[2] < v
    assert cuda.tm_cuda_tok_begin()
    cuda.tm_cuda_tok_sample(LOGITS, TOK, 0, v, 1e4, 3)
    assert cuda.tm_cuda_tok_end(TOK, None, 0)
    assert int(down(cuda, TOK, 1, np.uint32)[0]) == 123456


def test_probe_copy_reads_registered_weights(cuda):
    W = synth.make_weights(synth.Q8_0, 4, 256, seed=3)
    wid, woff = wbuf(cuda, W)
    assert cuda.tm_cuda_tok_probe_copy(wid, 10, T1, 64), lib.last_error()
    assert np.array_equal(down(cuda, T1, 64, np.uint8), W.reshape(-1)[10:74])


@pytest.mark.parametrize("dh,pos", [(128, 0), (128, 31), (128, 32), (128, 257), (64, 100)])
def test_fused_chain_attention_equals_the_separate_launches(cuda, dh, pos):
    """tok_attn_fused_at (one launch) against tok_qkv_post_at + tok_attn_at on the same inputs: the caches
    receive bit-identical rows at the position, the outputs agree to fp32 rounding of a reordered sum."""
    Hh, KVH, ctx = 8, 2, 300
    QD, KVD = Hh * dh, KVH * dh
    g = np.random.default_rng(1234 + pos)
    qkv = g.standard_normal(QD + 2 * KVD).astype(np.float32)
    hist_k = g.standard_normal(KVH * ctx * dh).astype(np.float32)
    hist_v = g.standard_normal(KVH * ctx * dh).astype(np.float32)
    S_QKV, S_KC1, S_VC1, S_KC2, S_VC2, S_P1, S_P2, S_O1, S_O2, S_ST = range(40, 50)
    scale, theta = 1.0 / np.sqrt(dh), 500000.0
    for s in (S_KC1, S_KC2):
        assert cuda.tm_cuda_tok_kv_reserve(s, KVH * ctx * dh)
        lib.check(cuda.tm_cuda_tok_kv_upload(s, 0, hist_k.ctypes.data, hist_k.size), "kv_upload")
    for s in (S_VC1, S_VC2):
        assert cuda.tm_cuda_tok_kv_reserve(s, KVH * ctx * dh)
        lib.check(cuda.tm_cuda_tok_kv_upload(s, 0, hist_v.ctypes.data, hist_v.size), "kv_upload")
    assert cuda.tm_cuda_tok_reserve(S_QKV, qkv.nbytes) and cuda.tm_cuda_tok_reserve(S_ST, 64)
    assert cuda.tm_cuda_tok_reserve(S_O1, QD * 4) and cuda.tm_cuda_tok_reserve(S_O2, QD * 4)
    assert cuda.tm_cuda_tok_reserve(S_P1, Hh * ctx * 4) and cuda.tm_cuda_tok_reserve(S_P2, Hh * (dh + 2) * 4 * 80)
    up(cuda, S_ST, np.array([pos, 0, 0, 0], np.int32))
    # separate launches (they rotate q in place, so the fused call gets a fresh copy afterwards)
    up(cuda, S_QKV, qkv)
    assert cuda.tm_cuda_tok_begin()
    cuda.tm_cuda_tok_qkv_post_at(S_QKV, S_KC1, S_VC1, Hh, KVH, dh, ctx, theta, S_ST)
    cuda.tm_cuda_tok_attn_at(S_QKV, S_KC1, S_VC1, S_P1, S_O1, QD, Hh, KVH, dh, ctx, scale, Hh // KVH, S_ST)
    assert cuda.tm_cuda_tok_flush(), lib.last_error()
    up(cuda, S_QKV, qkv)
    assert cuda.tm_cuda_tok_begin()
    cuda.tm_cuda_tok_attn_fused_at(S_QKV, S_KC2, S_VC2, S_P2, S_O2, Hh, KVH, dh, ctx, scale, theta, S_ST)
    assert cuda.tm_cuda_tok_flush(), lib.last_error()
    o1, o2 = down(cuda, S_O1, QD), down(cuda, S_O2, QD)
    assert np.all(np.isfinite(o2))
    assert np.max(np.abs(o1 - o2)) <= 2e-5 * max(1.0, np.max(np.abs(o1)))
    for a, b in ((S_KC1, S_KC2), (S_VC1, S_VC2)):
        ka, kb = np.empty(KVH * ctx * dh, np.float32), np.empty(KVH * ctx * dh, np.float32)
        lib.check(cuda.tm_cuda_tok_kv_download(a, 0, ka.ctypes.data, ka.size), "kv_download")
        lib.check(cuda.tm_cuda_tok_kv_download(b, 0, kb.ctypes.data, kb.size), "kv_download")
        assert np.array_equal(ka.view(np.uint32), kb.view(np.uint32))


def test_tmq_container_to_lane(cuda, orc, tmp_path):
    """A .tmq file (records without padding, so payloads at odd offsets) -> one aligned weight handle -> GEMVs,
    single and segmented, equal to the oracle on the same bytes."""
    import struct

    from tensormark_b200 import chain as chain_mod
    k = 2048
    spec = [("blk.q", synth.Q4_0, 96), ("blk.k", synth.Q4_0, 32), ("blk.v", synth.Q4_0, 32), ("head", synth.Q6_K, 100)]
    out = [b"TMQ1", struct.pack("<I", len(spec))]
    Ws = {}
    for i, (name, dt, n) in enumerate(spec):
        W = synth.make_weights(dt, n, k, seed=300 + i)
        Ws[name] = W
        out += [struct.pack("<I", len(name)), name.encode(), struct.pack("<II", dt, 2), struct.pack("<II", n, k),
                struct.pack("<Q", n * k // synth.BLOCK_ELEMS[dt]), W.tobytes()]
    path = tmp_path / "model.tmq"
    path.write_bytes(b"".join(out))
    wid, info = chain_mod.tmq_upload(str(path), [s[0] for s in spec])
    assert wid >= 1000 and all(off % 256 == 0 for off, _, _ in info.values())
    x = synth.make_activations(k, seed=77)
    up(cuda, X, x)
    assert cuda.tm_cuda_tok_reserve(T1, 4 * 160)
    assert cuda.tm_cuda_tok_begin()
    offs = (C.c_uint64 * 3)(info["blk.q"][0], info["blk.k"][0], info["blk.v"][0])
    rows = (C.c_uint * 3)(96, 32, 32)
    cuda.tm_cuda_tok_gemv_seg_dt(X, wid, T1, 0, 160, k, synth.Q4_0, offs, rows, 3)
    assert cuda.tm_cuda_tok_flush(), lib.last_error()
    y = down(cuda, T1, 160)
    want = np.concatenate([orc.gemv_f64(synth.Q4_0, Ws[n], x, Ws[n].shape[0], k)[0] for n in ("blk.q", "blk.k", "blk.v")])
    wabs = np.concatenate([orc.gemv_f64(synth.Q4_0, Ws[n], x, Ws[n].shape[0], k)[1] for n in ("blk.q", "blk.k", "blk.v")])
    assert np.all(np.abs(y - want) <= 1e-3 * wabs)
    assert cuda.tm_cuda_tok_begin()
    cuda.tm_cuda_tok_gemv_kq(X, wid, info["head"][0], T1, 0, 100, k, synth.Q6_K)
    assert cuda.tm_cuda_tok_flush(), lib.last_error()
    y = down(cuda, T1, 100)
    want, wabs = orc.gemv_f64(synth.Q6_K, Ws["head"], x, 100, k)
    assert np.all(np.abs(y - want) <= 1e-3 * wabs)
