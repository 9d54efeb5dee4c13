"""A device-side wait on another GPU that never gets its signal must end by itself and report, not hang.

One GPU is enough: the peer arena is opened in its loopback form as rank 0 of 2, so rank 1's counters never
advance. A GEMV that consumes a "gathered" vector then waits for rank 1, runs into the (shortened) limit, goes
on, and the next synchronising entry returns false with the status named in the message. The first expiry
raises the arena's abort word: the other waits of the same token return at once, so three waiting kernels cost
one limit, not three. Nothing faults or traps; the lane is usable afterwards.
(The reference's analogue is the 30 s deadline of its GPU/CPU hand-off, tensormark/metal_llama.h:856-876.)"""
import ctypes as C
import time

import numpy as np
import pytest

from tensormark_b200 import lib, synth

pytestmark = pytest.mark.gpu

XS, YS, ZS, ST = 60, 61, 62, 63          # slot ids of this test only


def test_wait_limit_expires_reports_and_recovers(cuda):
    L = cuda
    n, k, dt = 512, 2048, synth.Q4_0
    W = synth.make_weights(dt, n, k, seed=70)
    x = synth.make_activations(k, seed=71)
    handle = (C.c_ubyte * int(L.tm_cuda_peer_handle_bytes()))()
    assert L.tm_cuda_peer_arena(1 << 20, handle), lib.last_error()
    limit_ms = 150
    prev = L.tm_cuda_set_wait_limit_ms(limit_ms)
    try:
        assert L.tm_cuda_peer_open_loopback(0, 2), lib.last_error()
        assert L.tm_cuda_tok_reserve(XS, 4 * k) and L.tm_cuda_tok_reserve(ZS, 4 * n) and L.tm_cuda_tok_reserve(ST, 64)
        assert L.tm_cuda_tok_reserve_shared(YS, 4 * n), lib.last_error()
        state = np.zeros(4, np.int32)
        assert L.tm_cuda_tok_upload(ST, 0, state.ctypes.data, 16) and L.tm_cuda_tok_upload(XS, 0, x.ctypes.data, x.nbytes)
        woff = C.c_uint64(0)
        wid = L.tm_cuda_tok_wbuf(W.ctypes.data, W.nbytes, None, 0, 0, C.byref(woff))
        assert wid >= 1000, lib.last_error()
        seg_woff, seg_rows, seg_yoff = (C.c_uint64 * 1)(woff.value), (C.c_uint * 1)(n), (C.c_size_t * 1)(0)

        def gemv(yslot, wait_site, push_site):
            L.tm_cuda_tok_gemv_xchg(XS, 0, 0, 0, 0, None, 0.0, wid, yslot, seg_yoff, n, k, dt, seg_woff, seg_rows, 1, 0,
                                    wait_site, push_site, ST)

        # a producer only pushes (its rows and its count land in this GPU's own arena): nothing to wait for
        assert L.tm_cuda_tok_begin()
        gemv(YS, -1, 5)
        assert L.tm_cuda_tok_flush(), lib.last_error()
        want = np.empty(n, np.float32)
        assert L.tm_cuda_tok_download(YS, 0, want.ctypes.data, want.nbytes)

        # three consumers of site 5 wait for rank 1, which does not exist
        fb = int(L.tm_cuda_fallback_count())
        assert L.tm_cuda_tok_begin()
        t0 = time.perf_counter()
        for _ in range(3):
            gemv(ZS, 5, -1)
        ok = L.tm_cuda_tok_flush()
        took = time.perf_counter() - t0
        assert not ok
        assert "bounded wait" in lib.last_error() and "status 2" in lib.last_error()
        assert int(L.tm_cuda_fallback_count()) > fb
        assert limit_ms * 1e-3 * 0.5 <= took < limit_ms * 1e-3 * 2.5, took      # one limit, not three; and no hang
        got = np.empty(n, np.float32)
        assert L.tm_cuda_tok_download(ZS, 0, got.ctypes.data, got.nbytes)
        assert np.array_equal(got, want)             # the kernels went on after giving up (the data happened to be there)

        # the status and the abort word are cleared: launches without a wait are clean again
        assert L.tm_cuda_tok_begin()
        gemv(YS, -1, 5)
        assert L.tm_cuda_tok_flush(), lib.last_error()
    finally:
        L.tm_cuda_set_wait_limit_ms(prev)
        L.tm_cuda_peer_unmap()
        L.tm_cuda_peer_close()
