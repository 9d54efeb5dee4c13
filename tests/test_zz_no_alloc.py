"""The allocation-free decode attention entry against the ordinary one.

Collected last on purpose (file name): if it fails, a run that stops at the first failure has
already executed every other test. The entry under test keeps its split-K scratch in a static
device array, for hosts that have no device memory left to allocate from or cannot afford an
allocation on their token path; it must give what tm_cuda_attn_decode_dev gives, call after call,
although both calls write the same array."""
from __future__ import annotations

import numpy as np
import pytest

from tensormark_b200 import lib
from tests.gpu_util import ptr, stream_ptr

pytestmark = pytest.mark.gpu


def _case(torch, Hn, KVH, dh, ctx, seed, half):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(Hn * dh, generator=g, device="cuda", dtype=torch.float32)
    k = torch.randn(KVH * ctx * dh, generator=g, device="cuda", dtype=torch.float32)
    v = torch.randn(KVH * ctx * dh, generator=g, device="cuda", dtype=torch.float32)
    if half:
        k, v = k.half(), v.half()
    return q, k, v


@pytest.mark.parametrize("half", [1, 0])
def test_static_scratch_attention_matches_twice_in_a_row(cuda, torch_mod, half):
    torch = torch_mod
    Hn, KVH, dh, ctx = 32, 8, 128, 1024          # the decode-chain head geometry
    scale = 1.0 / np.sqrt(dh)
    sp = stream_ptr(torch)
    for call, allow in enumerate((640, 97)):      # two calls in a row share the array; the second is shorter
        q, k, v = _case(torch, Hn, KVH, dh, ctx, 20 + call, half)
        need = cuda.tm_cuda_attn_decode_scratch(Hn, KVH, dh, ctx, allow)
        scratch = torch.empty(need // 4 + 4, dtype=torch.float32, device="cuda")
        want = torch.empty(Hn * dh, dtype=torch.float32, device="cuda")
        got = torch.full((Hn * dh,), float("nan"), dtype=torch.float32, device="cuda")
        lib.check(cuda.tm_cuda_attn_decode_dev(ptr(q), ptr(k), ptr(v), ptr(scratch), need, ptr(want), Hn, KVH, dh, ctx,
                                               allow, scale, half, sp), "tm_cuda_attn_decode_dev")
        before = torch.cuda.memory_allocated()
        lib.check(cuda.tm_cuda_attn_decode_static_dev(ptr(q), ptr(k), ptr(v), ptr(got), Hn, KVH, dh, ctx, allow, scale,
                                                      half, sp), "tm_cuda_attn_decode_static_dev")
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        # the tolerance the attention parity tests use (1e-3 relative, 2e-5 absolute)
        assert np.allclose(got.cpu().numpy(), want.cpu().numpy(), rtol=1e-3, atol=2e-5)


def test_static_scratch_refuses_what_does_not_fit(cuda, torch_mod):
    torch = torch_mod
    Hn, KVH, dh, ctx, allow = 64, 8, 128, 1024, 1024      # 19 splits x 64 heads x 130 floats = 632 KB > 512 KB
    q, k, v = _case(torch, Hn, KVH, dh, ctx, 3, 1)
    out = torch.zeros(Hn * dh, dtype=torch.float32, device="cuda")
    before = cuda.tm_cuda_fallback_count()
    assert not cuda.tm_cuda_attn_decode_static_dev(ptr(q), ptr(k), ptr(v), ptr(out), Hn, KVH, dh, ctx, allow, 0.1, 1,
                                                   stream_ptr(torch))
    assert cuda.tm_cuda_fallback_count() == before + 1
    assert "static array holds" in lib.last_error()
    torch.cuda.synchronize()
    assert not out.any()                                   # nothing ran
