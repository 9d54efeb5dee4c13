"""GPU decode chain (C++ driver over the token lane) against the CPU chain, teacher-forced.

Random-init weights give near-flat logits, so a free-running greedy trajectory is knife-edged; parity
is therefore judged on logits with both sides fed the same tokens (the reference's own GPU-vs-CPU bar:
1e-3 with fp32 glue, test_llama_gpu_stack.cpp:10-14), and the lanes of the driver are compared with
each other on tokens (chain vs host loop must give identical tokens, test_llama_gpu_stack.cpp:57-76)."""
from __future__ import annotations

import numpy as np
import pytest

from oracle import binding
from tensormark_b200 import chain, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tiny():
    cfg = dict(synth.TINY_CHAIN)
    w = synth.make_llama(cfg, seed=5)
    return cfg, w


def _tol(ref):
    return 1e-3 * max(1.0, float(np.abs(ref).max()))


def test_forward_matches_cpu_chain_teacher_forced(cuda, orc, tiny):
    cfg, w = tiny
    cpu = binding.ChainModel(orc, cfg, w, kv_half=True)      # the GPU cache stores K/V rows as half by default
    gpu = chain.Chain(cfg, w)
    toks = synth.make_tokens(24, cfg["V"], seed=5)
    for pos, t in enumerate(toks):
        want = cpu.step(int(t), pos)
        got = gpu.forward(int(t))
        assert gpu.seen == pos + 1
        assert np.abs(got - want).max() <= _tol(want), pos
    # the three lanes from the same state: host loop of forwards, reference-order chain, graph chain
    first = int(toks[-1])
    base = gpu.seen
    n = 12
    loop_tokens, t = [], first
    for i in range(n):
        t = int(np.argmax(gpu.forward(t)))
        loop_tokens.append(t)
    loop_logits_seen = gpu.seen
    gpu.seen = base
    ref_tokens, ref_logits = gpu.greedy(first, n, graph=False)
    assert gpu.seen == loop_logits_seen
    assert list(ref_tokens) == loop_tokens                   # same kernels, same order: identical tokens
    gpu.seen = base
    g_tokens, g_logits = gpu.greedy(first, n, graph=True)
    assert list(g_tokens) == loop_tokens
    assert np.abs(g_logits - ref_logits).max() <= _tol(ref_logits)
    # a second graph chain reuses the captured graph and continues from the new position
    more, _ = gpu.greedy(int(g_tokens[-1]), 5, graph=True)
    cpu_tokens, t = [], int(g_tokens[-1])
    # bring the CPU chain to the same state (feed what the GPU fed), then compare the continuation's logits
    fed = [first] + loop_tokens[:-1]
    for i, tk in enumerate(fed):
        cpu.step(tk, base + i)
    for i in range(5):
        lg = cpu.step(t, base + n + i)
        cpu_tokens.append(int(np.argmax(lg)))
        t = int(more[i])                                     # teacher-forced with the GPU's choice
        top2 = np.sort(lg)[-2:]
        if cpu_tokens[-1] != int(more[i]):
            assert top2[1] - top2[0] <= _tol(lg)             # a different choice is only acceptable on a numerical tie
    gpu.close()


def test_prompt_feed_equals_forward_loop(cuda, tiny):
    cfg, w = tiny
    toks = synth.make_tokens(20, cfg["V"], seed=9).astype(np.int32)
    a = chain.Chain(cfg, w)
    last = None
    for t in toks:
        last = a.forward(int(t))
    nxt_loop = int(np.argmax(last))
    cont_loop, _ = a.greedy(nxt_loop, 6, graph=False)
    a.close()
    b = chain.Chain(cfg, w)
    nxt = b.feed(toks)
    assert b.seen == len(toks) and nxt == nxt_loop
    cont, _ = b.greedy(nxt, 6, graph=True)
    assert list(cont) == list(cont_loop)
    b.close()


def test_chain_polling_and_argument_errors(cuda, tiny):
    cfg, w = tiny
    gpu = chain.Chain(cfg, w, shared_mapping=False)          # one device copy per tensor: no fused segments
    gpu.forward(3)
    gpu.chain_begin(7, 6, graph=False)
    got = gpu.chain_end(6)
    assert len(got) == 6 and all(0 <= int(t) < cfg["V"] for t in got)
    assert gpu.chain_poll(0) == -1                            # no chain running
    gpu.chain_begin(int(got[-1]), 4, graph=True)
    out = gpu.chain_end(4, keep=1)                            # stopped at chosen token 1: position = start + 2
    assert len(out) == 4 and gpu.seen == 1 + 6 + 2
    with pytest.raises(RuntimeError):
        gpu.chain_begin(1, 0)                                 # n >= 1
    with pytest.raises(RuntimeError):
        gpu.chain_begin(1, cfg["ctx"])                        # exceeds the context
    with pytest.raises(RuntimeError):
        gpu.forward(cfg["V"])                                 # token id out of range
    gpu.close()


def _gumbel_choice(logits: np.ndarray, idx: int, inv_temp: float, seed: int) -> int:
    """The reference's sampler restated with numpy (tensormark/metal.h:2349-2379): noise = hash(seed, idx, i)."""
    def h32(x):
        x = x.astype(np.uint64) & 0xFFFFFFFF
        x ^= x >> 16; x = (x * 0x7feb352d) & 0xFFFFFFFF
        x ^= x >> 15; x = (x * 0x846ca68b) & 0xFFFFFFFF
        x ^= x >> 16
        return x
    base = h32(np.array([(seed * 0x9e3779b9 + idx * 0x85ebca6b + 0x1234567) & 0xFFFFFFFF], dtype=np.uint64))[0]
    i = np.arange(logits.size, dtype=np.uint64)
    h = h32(np.uint64(base) ^ ((i * 0x27d4eb2f + 0x165667b1) & 0xFFFFFFFF))
    u = ((h >> 8).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
    v = logits.astype(np.float32) * np.float32(inv_temp) - np.log(-np.log(u.astype(np.float64))).astype(np.float32)
    return int(np.argmax(v)), np.sort(v)[-2:]


def test_sampled_chain(cuda, tiny):
    cfg, w = tiny
    a = chain.Chain(cfg, w)
    logits = a.forward(5)                                     # position 0; the chain below re-feeds token 5 at position 1
    a.seen = 0
    a.chain_begin_sampled(5, 6, 1.3, 77, graph=True)
    ta = a.chain_end(6)
    a.seen = 0
    a.chain_begin_sampled(5, 6, 1.3, 77, graph=False)        # one lane call per op, reference order
    tb = a.chain_end(6)
    assert list(ta) == list(tb)
    # first sampled token against the reference's formula on the same logits (index 1 of the token slot)
    want, top2 = _gumbel_choice(logits, 1, 1.3, 77)
    assert int(ta[0]) == want or abs(float(top2[1] - top2[0])) < 1e-4
    # another seed or temperature is another graph; a very low temperature is the greedy chain
    a.seen = 0
    a.chain_begin_sampled(5, 6, 1.3, 78, graph=True)
    tc = a.chain_end(6)
    a.seen = 0
    a.chain_begin_sampled(5, 6, 1e4, 78, graph=True)
    td = a.chain_end(6)
    a.seen = 0
    a.chain_begin(5, 6, graph=True)
    te = a.chain_end(6)
    assert list(td) == list(te)
    assert list(tc) != list(ta) or list(tc) != list(te)       # 6 draws from 1024 tokens at T = 0.77: not all equal by chance
    with pytest.raises(RuntimeError):
        a.chain_begin_sampled(5, 2, 0.0, 1)
    a.close()
