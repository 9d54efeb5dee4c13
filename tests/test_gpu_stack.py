"""The GPU prefill layer stack (include/llama_gpu_api.h) against the CPU block loop.

Mirrors the reference's own gate (tensormark/test_llama_gpu_stack.cpp): the stack's residual stream and every K/V
row it writes against the CPU path on the same tokens, at T = 8 (one query block) and T = 300 (several blocks), a
chunked prefill (200, then 100 more at position 200), bars below (the reference's: test_llama_gpu_stack.cpp:10-14); then
the begin / wait_layer / end form, the argument errors, and the hand-over of the prefilled rows to the decode lane.
The CPU side is oracle/tm_oracle.c's block loop (tmo_chain_step), one token at a time."""
from __future__ import annotations

import numpy as np
import pytest

from oracle import binding
from tensormark_b200 import chain, lib, stack, synth

pytestmark = pytest.mark.gpu

# two geometries: the tiny chain model (dh 64, REP 2) and a GQA model with config 5's head shape (dh 128, REP 4)
GQA128 = dict(L=2, D=512, H=8, KVH=2, dh=128, F=1024, V=512, ctx=320, theta=500000.0, eps=1e-5,
              dt_proj=synth.Q4_0, dt_head=synth.Q6_K, dt_embed=synth.Q4_0)
TINY = dict(synth.TINY_CHAIN, ctx=320)


def _embed(orc, cfg, w, toks):
    D = cfg["D"]
    return np.stack([orc.dequant(cfg["dt_embed"], w["embed"][int(t)], D) for t in toks]).astype(np.float32)


def _cpu_rows(orc, cfg, w, toks, pos0, cpu=None, biases=None):
    """Residual stream after the last layer for every token, through the CPU block loop; returns (rows, model)."""
    cpu = cpu or binding.ChainModel(orc, cfg, w, kv_half=False, threads=4, biases=biases)
    D = cfg["D"]
    out = np.empty((len(toks), D), np.float32)
    for i, t in enumerate(toks):
        _, taps = cpu.step(int(t), pos0 + i, tap_layer=cfg["L"] - 1)
        out[i] = taps[-D:]
    return out, cpu


# Bars. The reference's are 1e-3 for fp32 glue around fp32 GEMMs and 5e-2 (plus the same argmax) once activations
# between GEMMs are half (test_llama_gpu_stack.cpp:10-14). This stack keeps fp32 glue and fp32 accumulation but feeds
# the tensor cores fp16 operands (each weight and each activation rounded once, relative error 2^-11): K/V rows, one
# GEMM deep in the first layer, meet 1e-3; the residual stream after every layer is held to 5e-3 of its largest value.
ROW_BAR, STREAM_BAR = 1e-3, 5e-3


def _close(got, want, what, bar=ROW_BAR):
    scale = max(1.0, float(np.abs(want).max()))
    err = float(np.abs(got - want).max()) / scale
    assert np.isfinite(got).all() and err <= bar, (what, err)
    return err


@pytest.mark.parametrize("cfg", [TINY, GQA128], ids=["dh64-rep2", "dh128-rep4"])
@pytest.mark.parametrize("T", [8, 300])
def test_stack_matches_cpu_block_loop(cuda, orc, cfg, T):
    w = synth.make_llama(cfg, seed=21)
    toks = synth.make_tokens(T, cfg["V"], seed=22)
    want, cpu = _cpu_rows(orc, cfg, w, toks, 0)
    st = stack.Stack(cfg, w)
    got = st.prefill(_embed(orc, cfg, w, toks), 0)
    _close(got, want, "residual stream", STREAM_BAR)
    for l in (0, cfg["L"] - 1):                         # K/V rows of the first and the last layer, as the reference checks
        _close(st.kc[l][:, :T], cpu.kc[l][:, :T], f"K rows layer {l}", ROW_BAR if l == 0 else STREAM_BAR)
        _close(st.vc[l][:, :T], cpu.vc[l][:, :T], f"V rows layer {l}", ROW_BAR if l == 0 else STREAM_BAR)
        assert not st.kc[l][:, T:].any()                 # rows beyond the batch are untouched
    assert st.gpu_ms() > 0
    st.close()


@pytest.mark.parametrize("cfg", [TINY, GQA128], ids=["dh64-rep2", "dh128-rep4"])
def test_resident_fp16_weights_equal_per_call_conversion(cuda, orc, cfg, monkeypatch):
    """The stack keeps fp16 copies of its weights when they fit (q|k|v and gate|up then run as one GEMM each); with
    TM_CUDA_STACK_FP16=0 every GEMM call converts its weights again. Same fp16 operands, same order of accumulation over
    K for every output element: the two forms must agree bit for bit."""
    T = 300
    w = synth.make_llama(cfg, seed=23)
    x = _embed(orc, cfg, w, synth.make_tokens(T, cfg["V"], seed=24))
    out = []
    for mode in ("0", "1"):
        monkeypatch.setenv("TM_CUDA_STACK_FP16", mode)
        st = stack.Stack(cfg, w)
        got = st.prefill(x, 0)
        out.append((got, [k.copy() for k in st.kc], [v.copy() for v in st.vc]))
        st.close()
    assert np.array_equal(out[0][0].view(np.uint32), out[1][0].view(np.uint32))
    for a, b in zip(out[0][1] + out[0][2], out[1][1] + out[1][2]):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("cfg", [TINY, GQA128], ids=["dh64-rep2", "dh128-rep4"])
def test_attention_on_fp16_rows_and_on_tf32_rows(cuda, orc, cfg, monkeypatch):
    """The attention reads fp16 copies of the cache rows (m16n8k16 MMAs); TM_CUDA_STACK_ATTN=tf32 runs it on the fp32 rows
    rounded to tf32 instead. Both meet the CPU block loop, whole and chunked (the second chunk's earlier rows come back
    from the caller's arrays and are converted again), and they differ from each other by less than either bar."""
    T = 300
    w = synth.make_llama(cfg, seed=29)
    toks = synth.make_tokens(T, cfg["V"], seed=30)
    x = _embed(orc, cfg, w, toks)
    want, _ = _cpu_rows(orc, cfg, w, toks, 0)
    got = {}
    for mode in ("fp16", "tf32"):
        monkeypatch.setenv("TM_CUDA_STACK_ATTN", mode)
        st = stack.Stack(cfg, w)
        whole = st.prefill(x, 0)
        st.close()
        st = stack.Stack(cfg, w)
        a = st.prefill(x[:200], 0)
        b = st.prefill(x[200:], 200)
        st.close()
        _close(whole, want, f"{mode}: residual stream", STREAM_BAR)
        assert np.array_equal(a.view(np.uint32), whole[:200].view(np.uint32)), mode
        _close(b, whole[200:], f"{mode}: second chunk", ROW_BAR)
        got[mode] = whole
    _close(got["fp16"], got["tf32"], "fp16 rows against tf32 rows", ROW_BAR)


def test_device_only_caches_and_prompt_after_decode_steps(cuda, orc):
    """kc = vc = NULL keeps the K/V rows on the device: same residual stream, chunks continue from the device rows. And a
    prompt that follows tokens of the decode lane (whose rows the stack does not have) must still give the decode lane's
    answer: the chain driver then feeds it token by token."""
    cfg = GQA128
    w = synth.make_llama(cfg, seed=25)
    toks = synth.make_tokens(300, cfg["V"], seed=26)
    x = _embed(orc, cfg, w, toks)
    ref = stack.Stack(cfg, w)
    want = ref.prefill(x, 0)
    ref.close()
    st = stack.Stack(cfg, w, device_only=True)
    a = st.prefill(x[:200], 0)
    b = st.prefill(x[200:], 200)
    st.close()
    assert np.array_equal(a.view(np.uint32), want[:200].view(np.uint32))
    _close(b, want[200:], "second chunk on device rows", STREAM_BAR)
    cfg2 = dict(synth.TINY_CHAIN)
    w2 = synth.make_llama(cfg2, seed=5)
    t2 = synth.make_tokens(40, cfg2["V"], seed=33).astype(np.int32)
    one = chain.Chain(cfg2, w2)
    nxt_one = one.feed(t2)
    lg_one = one.logits()
    one.close()
    two = chain.Chain(cfg2, w2)
    two.prefill(t2[:20])                                  # through the stack
    two.feed(t2[20:25])                                   # decode lane: the stack's caches do not see these rows
    nxt_two = two.prefill(t2[25:])                        # must not use the stack's stale rows
    lg_two = two.logits()
    two.close()
    scale = max(1.0, float(np.abs(lg_one).max()))
    assert float(np.abs(lg_one - lg_two).max()) <= 2e-3 * scale
    assert nxt_one == nxt_two or np.sort(lg_one)[-1] - np.sort(lg_one)[-2] <= 2e-3 * scale


def test_residual_stream_gathered_on_the_device(cuda, orc):
    """prefill_begin_tokens embeds the tokens on the device (rows of the block-quantized table, dequantized exactly): the
    K/V rows of every layer must equal those of the same batch uploaded as host rows, bit for bit."""
    cfg = GQA128
    w = synth.make_llama(cfg, seed=27)
    toks = synth.make_tokens(150, cfg["V"], seed=28)
    a = stack.Stack(cfg, w)
    a.prefill(_embed(orc, cfg, w, toks), 0)
    b = stack.Stack(cfg, w)
    b.begin_tokens(toks, 0)
    assert b.end(), lib.last_error()
    for l in range(cfg["L"]):
        assert np.array_equal(a.kc[l].view(np.uint32), b.kc[l].view(np.uint32)), l
        assert np.array_equal(a.vc[l].view(np.uint32), b.vc[l].view(np.uint32)), l
    bad = toks.copy()
    bad[3] = cfg["V"]
    with pytest.raises(RuntimeError):
        b.begin_tokens(bad, 0)
    a.close()
    b.close()


def test_chunked_prefill_and_wait_layer(cuda, orc):
    cfg = GQA128
    w = synth.make_llama(cfg, seed=23)
    toks = synth.make_tokens(300, cfg["V"], seed=24)
    want_a, cpu = _cpu_rows(orc, cfg, w, toks[:200], 0)
    want_b, cpu = _cpu_rows(orc, cfg, w, toks[200:], 200, cpu=cpu)
    st = stack.Stack(cfg, w, shared_mapping=False)      # one device copy per tensor
    x = _embed(orc, cfg, w, toks)
    _close(st.prefill(x[:200], 0), want_a, "first chunk", STREAM_BAR)
    # second chunk through begin / wait_layer / end: layer l's rows are in the caller's arrays once wait_layer(l) returns
    st.begin(x[200:], 200)
    for l in range(cfg["L"]):
        assert st.wait_layer(l)
        _close(st.kc[l][:, 200:300], cpu.kc[l][:, 200:300], f"K rows layer {l} after wait_layer", ROW_BAR if l == 0 else STREAM_BAR)
        _close(st.vc[l][:, 200:300], cpu.vc[l][:, 200:300], f"V rows layer {l} after wait_layer", ROW_BAR if l == 0 else STREAM_BAR)
    assert not st.wait_layer(cfg["L"])                   # no such layer
    assert st.end()
    # the blocking form at the same position gives the residual stream (begin does not write x back)
    _close(st.prefill(x[200:], 200), want_b, "second chunk", STREAM_BAR)
    # rows [0, pos0) come from the CALLER's arrays: change one and the result must move
    st.kc[0][:, :200] *= 1.5
    moved = st.prefill(x[200:], 200)
    assert float(np.abs(moved - want_b).max()) > 2 * STREAM_BAR * max(1.0, float(np.abs(want_b).max()))
    st.close()


def test_stack_bias_other_format_and_errors(cuda, orc):
    cfg = dict(TINY, dt_proj=synth.Q8_0)                 # the reference's stack is Q4_0-only; this one takes the dtype
    w = synth.make_llama(cfg, seed=25)
    g = synth.rng_for(26, 5)
    QD, KVD = cfg["H"] * cfg["dh"], cfg["KVH"] * cfg["dh"]
    biases = {}
    for l in range(cfg["L"]):
        biases[f"l{l}.q_bias"] = g.standard_normal(QD).astype(np.float32) * 0.1
        biases[f"l{l}.k_bias"] = g.standard_normal(KVD).astype(np.float32) * 0.1
        biases[f"l{l}.v_bias"] = g.standard_normal(KVD).astype(np.float32) * 0.1
    toks = synth.make_tokens(40, cfg["V"], seed=27)
    want, cpu = _cpu_rows(orc, cfg, w, toks, 0, biases=biases)
    st = stack.Stack(cfg, w, biases=biases)
    x = _embed(orc, cfg, w, toks)
    # random Q8_0 blocks drive the residual stream to several hundred within two layers and make the softmax sharp: the
    # same operand rounding moves this composite twice as far as the Q4_0 models above
    _close(st.prefill(x, 0), want, "residual stream with attention bias", 2 * STREAM_BAR)
    L = cuda
    fb = int(L.tm_cuda_fallback_count())
    one = np.zeros((1, cfg["D"]), np.float32)
    assert not L.tm_cuda_llama_prefill(st.h, one.ctypes.data, 1, 0)                    # T >= 2 (metal_llama.h:899)
    assert not L.tm_cuda_llama_prefill(st.h, x.ctypes.data, 40, cfg["ctx"] - 39)       # beyond the context
    assert not L.tm_cuda_llama_prefill(st.h, x.ctypes.data, 40, -1)
    assert not L.tm_cuda_llama_prefill(None, x.ctypes.data, 40, 0)
    assert int(L.tm_cuda_fallback_count()) >= fb + 4
    assert L.tm_cuda_llama_create(None) is None
    st.close()


def test_prefill_hands_over_to_the_decode_chain(cuda, orc):
    """A prompt through the stack, its K/V rows moved into the decode lane on the device, then the greedy chain: the same
    tokens as feeding the prompt one token at a time through the decode lane."""
    cfg = dict(synth.TINY_CHAIN)
    w = synth.make_llama(cfg, seed=5)
    toks = synth.make_tokens(40, cfg["V"], seed=31).astype(np.int32)
    a = chain.Chain(cfg, w)
    nxt_a = a.feed(toks)
    cont_a, logits_a = a.greedy(nxt_a, 8)
    a.close()
    b = chain.Chain(cfg, w)
    nxt_b = b.prefill(toks)
    assert b.seen == len(toks)
    cont_b, logits_b = b.greedy(nxt_b, 8)
    b.close()
    scale = max(1.0, float(np.abs(logits_a).max()))
    if nxt_a == nxt_b and list(cont_a) == list(cont_b):
        assert float(np.abs(logits_a - logits_b).max()) <= 2e-3 * scale
    else:
        # the two paths round differently (fp16 GEMM operands against the GEMV's fixed-point activations): a different
        # choice is acceptable only on a numerical tie, checked on the CPU chain's logits for the prompt
        cpu = binding.ChainModel(orc, cfg, w, kv_half=True)
        lg = None
        for i, t in enumerate(toks):
            lg = cpu.step(int(t), i)
        top2 = np.sort(lg)[-2:]
        assert nxt_a == nxt_b or (top2[1] - top2[0]) <= 2e-3 * scale
