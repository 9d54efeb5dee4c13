"""CPU, two gloo ranks: the row-sharded GEMV (each rank its rows, all-gather of the outputs) equals the
unsharded one bit for bit, and small tensors stay replicated."""
from __future__ import annotations

import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank: int, world: int, port: int, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from oracle import binding
    from tensormark_b200 import shard, synth
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    orc = binding.oracle()
    ok = True
    for dt, n, k in [(synth.Q8_0, 4096, 512), (synth.Q6_K, 8192, 256), (synth.Q4_0, 256, 512)]:
        W = synth.make_weights(dt, n, k, seed=31)
        x = synth.make_activations(k, seed=32)
        lo, hi = shard.row_range(n, rank, world)
        part = torch.from_numpy(orc.gemv(dt, W[lo:hi], x, hi - lo, k))
        if shard.is_sharded(n, world):
            full = torch.empty(n, dtype=torch.float32)
            dist.all_gather_into_tensor(full, part)
        else:
            full = part
            ok = ok and (lo, hi) == (0, n)
        ref = orc.gemv(dt, W, x, n, k)
        ok = ok and np.array_equal(full.numpy().view(np.uint32), ref.view(np.uint32))
    # max-over-ranks timing reduction, as the benchmark does it
    t = torch.tensor([float(rank + 1)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = ok and t.item() == float(world)
    dist.destroy_process_group()
    q.put((rank, ok))


def test_row_sharded_gemv_two_ranks():
    import torch.multiprocessing as mp
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, True), (1, True)]


def test_row_range_arithmetic():
    from tensormark_b200 import shard
    assert shard.row_range(32000, 3, 8) == (12000, 16000)
    assert shard.row_range(5632, 1, 2) == (2816, 5632)
    assert shard.row_range(2048, 1, 2) == (0, 2048)          # below the threshold: replicated
    assert shard.row_range(128256, 7, 8) == (112224, 128256)
    assert shard.row_range(4097, 0, 2) == (0, 4097)          # does not divide: replicated
    covered = sorted(shard.row_range(14336, r, 4) for r in range(4))
    assert covered[0][0] == 0 and covered[-1][1] == 14336 and all(a[1] == b[0] for a, b in zip(covered, covered[1:]))
    with pytest.raises(ValueError):
        shard.row_range(8192, 2, 2)
