"""The choice of a row-sharded LM head that exchanges (value, index) keys instead of logits (tm_cuda_tok_choose_shard).

One GPU is enough to pin its arithmetic: the peer arena is opened in loopback as one rank of two, and the test plays the
other rank - it writes that rank's key into the key table and advances its counter (tm_cuda_peer_bump), as the other
rank's kernel would. The winner must be the token the unsharded choice takes over the whole vector: largest value,
lowest index on ties (tensormark/metal.h:2335), and with a temperature the Gumbel-max of the reference's sampler
(tensormark/metal.h:2349-2379) with the noise of the GLOBAL row index. Two GPUs run the real exchange in
tests/test_gpu_shard.py."""
import ctypes as C

import numpy as np
import pytest

from tensormark_b200 import lib
from tests.test_gpu_chain import _gumbel_choice

pytestmark = pytest.mark.gpu

XS, TK, ST, KS = 64, 65, 66, 67          # slot ids of this test only
V, HALF, SITE = 4000, 2000, 9


def pack_key(v: float, i: int) -> int:
    """The kernel's 64-bit key: unsigned order = larger value first, then lower index."""
    b = int(np.float32(v).view(np.uint32))
    b = (~b & 0xFFFFFFFF) if b & 0x80000000 else (b | 0x80000000)
    return (b << 32) | (0xFFFFFFFF - i)


def gumbel_values(logits: np.ndarray, idx: int, inv_temp: float, seed: int) -> np.ndarray:
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
    return logits.astype(np.float32) * np.float32(inv_temp) - np.log(-np.log(u.astype(np.float64))).astype(np.float32)


class Rehearsal:
    """This process as rank `rank` of 2 on a loopback arena; `other` is the rank the test plays."""

    def __init__(self, L, rank: int):
        self.L, self.rank, self.other, self.step = L, rank, 1 - rank, 0
        handle = (C.c_ubyte * int(L.tm_cuda_peer_handle_bytes()))()
        assert L.tm_cuda_peer_arena(1 << 20, handle), lib.last_error()
        assert L.tm_cuda_peer_open_loopback(rank, 2), lib.last_error()
        assert L.tm_cuda_tok_reserve(XS, 4 * V) and L.tm_cuda_tok_reserve(TK, 4 * 64) and L.tm_cuda_tok_reserve(ST, 64)
        assert L.tm_cuda_tok_reserve_shared(KS, 16), lib.last_error()
        state = np.zeros(4, np.int32)
        assert L.tm_cuda_tok_upload(ST, 0, state.ctypes.data, 16)

    def choose(self, logits: np.ndarray, other_key: int | None, inv_temp: float = 0.0, seed: int = 0, bump: int = 1) -> tuple[bool, int]:
        """One token: the other rank's key and count are in place (or not) before this rank's kernel waits for them."""
        L = self.L
        assert L.tm_cuda_tok_upload(XS, 0, logits.ctypes.data, logits.nbytes)
        if other_key is not None:
            key = np.array([other_key], np.uint64)
            assert L.tm_cuda_tok_upload(KS, 8 * self.other, key.ctypes.data, 8)
            assert L.tm_cuda_peer_bump(SITE, self.other, bump), lib.last_error()
        assert L.tm_cuda_tok_begin()
        L.tm_cuda_tok_choose_shard(XS, self.rank * HALF, HALF, V, TK, 64, inv_temp, seed, ST, KS, SITE)
        L.tm_cuda_tok_advance(ST)
        ok = bool(L.tm_cuda_tok_flush())
        self.step += 1
        tok = np.zeros(1, np.uint32)
        assert L.tm_cuda_tok_download(TK, 4 * self.step, tok.ctypes.data, 4)      # the entry the NEXT step would feed
        return ok, int(tok[0])

    def close(self):
        self.L.tm_cuda_peer_unmap()
        self.L.tm_cuda_peer_close()


def test_greedy_choice_over_two_shards(cuda):
    rng = np.random.default_rng(3)
    logits = rng.standard_normal(V).astype(np.float32)
    logits[777] = 5.0                                         # the largest value of rank 0's rows
    r = Rehearsal(cuda, 0)
    try:
        for other, want in (((4.0, 3100), 777),               # the other rank's best is smaller
                            ((9.0, 2500), 2500),              # ... larger
                            ((5.0, 2100), 777),               # ... equal: the lower index wins
                            ((float("-inf"), 0), 777)):       # ... nothing finite (its key is the kernel's initial one)
            ok, tok = r.choose(logits, pack_key(*other))
            assert ok, lib.last_error()
            assert tok == want, (other, tok)
    finally:
        r.close()
    # as the rank with the HIGHER rows: on equal values the other rank's lower index wins
    logits[777] = 0.0
    logits[2600] = 5.0
    r = Rehearsal(cuda, 1)
    try:
        ok, tok = r.choose(logits, pack_key(5.0, 1234))
        assert ok and tok == 1234, tok
        ok, tok = r.choose(logits, pack_key(4.999, 1234))
        assert ok and tok == 2600, tok
    finally:
        r.close()


def test_sampled_choice_uses_the_global_row_index(cuda):
    rng = np.random.default_rng(4)
    logits = (rng.standard_normal(V) * 2).astype(np.float32)
    inv_temp, seed = 1.3, 77
    for rank in (0, 1):
        r = Rehearsal(cuda, rank)
        try:
            for step in range(3):
                idx = step + 1                                 # the token slot entry this step writes
                v = gumbel_values(logits, idx, inv_temp, seed)
                lo = (1 - rank) * HALF                         # the OTHER rank's rows, reduced here as its kernel would
                j = lo + int(np.argmax(v[lo: lo + HALF]))
                ok, tok = r.choose(logits, pack_key(float(v[j]), j), inv_temp, seed)
                want, top2 = _gumbel_choice(logits, idx, inv_temp, seed)
                assert ok, lib.last_error()
                assert tok == want or abs(float(top2[1] - top2[0])) < 1e-4, (rank, step, tok, want)
        finally:
            r.close()


def test_missing_rank_runs_into_the_wait_limit(cuda):
    L = cuda
    logits = np.zeros(V, np.float32)
    prev = L.tm_cuda_set_wait_limit_ms(100)
    r = Rehearsal(L, 0)
    try:
        ok, _ = r.choose(logits, None)                         # nobody plays rank 1
        assert not ok and "status 2" in lib.last_error()
        ok, tok = r.choose(logits, pack_key(1.0, 3000), bump=2)     # the late rank catches up (two tokens' counts): clean again
        assert ok, lib.last_error()
        assert tok == 3000
    finally:
        L.tm_cuda_set_wait_limit_ms(prev)
        r.close()
