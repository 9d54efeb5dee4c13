"""Run one kernel of the path on a chosen shape, a few times, and print its timing.

    python -m tensormark_b200.run_case --op gemv --dtype Q8_0 --n 32000 --k 2048 --reps 5 --copies 3
    python -m tensormark_b200.run_case --op gemm --dtype Q4_0 --m 2000 --n 5632 --k 2048 --reps 3
    python -m tensormark_b200.run_case --op dequant --dtype Q6_K --n 4096 --k 4096

A small, self-contained driver for profilers and for tuning: it creates seeded synthetic
inputs on the device, launches the kernel through the C ABI on one stream and reports the
CUDA-event time per launch together with the algorithmic GB/s or TFLOP/s.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json

import numpy as np

from . import lib, synth

NAMES = {v: k for k, v in synth.DTYPE_NAMES.items()}


def cfg_for(args) -> dict:
    cfg = dict(synth.LLAMA3_8B if args.model == "llama3-8b" else synth.TINY_CHAIN)
    cfg["ctx"] = max(cfg["ctx"], args.prompt + args.steps + 1) if args.model == "llama3-8b" else cfg["ctx"]
    return cfg


def summarize_trace(L, per: int):
    """Per-shape averages of the library's kernel timeline (TM_CUDA_TRACE=1 in the environment) over the last
    tokens of the chain: for every GEMV the time from CTA start to the end of the wait for its predecessor, the
    x phase, the row phase and start -> end; for the fused attention its phases. None when tracing is off."""
    import collections
    cap = 8192
    buf = (C.c_ulonglong * (6 * cap))()
    n = int(L.tm_cuda_trace_read(buf, cap))
    if n == 0:
        return None
    a = np.frombuffer(buf, dtype=np.uint64)[: n * 6].reshape(n, 6).astype(np.int64)
    a = a[np.argsort(a[:, 0])]
    whole = n // per                                        # whole tokens in the log (it keeps the first 8192 launches)
    if whole == 0:
        return None
    tail = a[per * max(0, whole - 4): per * whole]
    agg = collections.defaultdict(lambda: [0, 0.0, 0.0, 0.0, 0.0])
    for r in tail:
        if r[5] >= r[0]:                                   # attention record: words 4 and 5 are timestamps
            g = agg["attn_fused"]
            g[0] += 1; g[1] += r[1] - r[0]; g[2] += r[2] - r[1]; g[3] += r[4] - r[2]; g[4] += r[5] - r[0]
        else:
            key = "gemv %dx%d dt%d xop%d" % (r[4] >> 32, r[4] & 0xffffffff, r[5] & 255, (r[5] >> 8) & 255)
            g = agg[key]
            g[0] += 1; g[1] += r[1] - r[0]; g[2] += r[2] - r[1]; g[3] += r[3] - r[2]; g[4] += r[3] - r[0]
    span = (tail[-1, 3] - tail[0, 0]) / 1e3 / max(1, len(tail) // per)
    return {"records": n, "launches_per_token": per, "token_span_us": round(float(span), 1),
            "per_kernel_us": {k: {"n": g[0], "wait": round(g[1] / g[0] / 1e3, 2), "x": round(g[2] / g[0] / 1e3, 2),
                                  "rows": round(g[3] / g[0] / 1e3, 2), "total": round(g[4] / g[0] / 1e3, 2)} for k, g in agg.items()}}


def chain_weight_bytes(cfg: dict) -> int:
    """Block bytes one token streams: every projection of every layer plus the LM head."""
    QD, KVD = cfg["H"] * cfg["dh"], cfg["KVH"] * cfg["dh"]
    per_layer = sum(synth.weight_bytes(cfg["dt_proj"], n, k) for n, k in
                    ((QD, cfg["D"]), (KVD, cfg["D"]), (KVD, cfg["D"]), (cfg["D"], QD), (cfg["F"], cfg["D"]), (cfg["F"], cfg["D"]), (cfg["D"], cfg["F"])))
    return cfg["L"] * per_layer + synth.weight_bytes(cfg["dt_head"], cfg["V"], cfg["D"])


def measure_chain(L, torch, cfg: dict, w: dict, prompt_n: int, steps: int, rank: int = 0, world: int = 1, gather: str = "peer",
                  dist=None, graph: bool = True, trace: bool = False, prefill: str = "feed") -> dict:
    """Feed `prompt_n` tokens, then time `steps` greedy tokens chosen on the GPU (CUDA events on the lane stream, max over
    ranks). world > 1: FFN and LM-head rows sharded over the ranks; the communicator (and, for gather == "peer", the peer
    arena) must exist already and `dist` is the initialised torch.distributed module (any backend). Returns the record
    every rank computes; "logits" (numpy) is the last step's logits of this rank."""
    import hashlib
    import time

    from . import chain
    cuda_group = dist is not None and dist.get_backend() == "nccl"

    def reduce(t, op):
        if cuda_group:
            t = t.cuda()
        dist.all_reduce(t, op=op)
        return t.cpu()

    m = chain.Chain(cfg, w, rank=rank, world=world, peer_gather=world > 1 and gather == "peer")
    prompt = synth.make_tokens(prompt_n, cfg["V"], seed=5).astype(np.int32)
    stream = torch.cuda.ExternalStream(L.tm_cuda_tok_stream())
    t0 = time.perf_counter()
    prefill_gpu_ms = None
    if prefill == "stack" and prompt_n >= 3:
        m.prefill_prepare(prompt_n)                        # one-time set-up (device caches, fp16 weight copies, batch buffers) is not prompt time
        t0 = time.perf_counter()
        nxt = m.prefill(prompt)                            # the batched layer stack (tensor-core GEMMs)
        prefill_gpu_ms = m.prefill_gpu_ms()
    elif not graph:
        last = None
        for t in prompt:
            last = m.forward(int(t))
        nxt = int(np.argmax(last))
    else:
        nxt = m.feed(prompt)
    t_prompt = time.perf_counter() - t0
    if graph:
        # one untimed token: the chain's CUDA graph exists afterwards whichever way the prompt went in
        one, _ = m.greedy(nxt, 1)
        nxt = int(one[0])
    if dist is not None and world > 1:
        dist.barrier()
    if trace:                                               # drop the prompt's records: the log holds 8192 launches
        L.tm_cuda_trace_read((C.c_ulonglong * (6 * 8192))(), 8192)
    launches0 = int(L.tm_cuda_launch_count())
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    t0 = time.perf_counter()
    m.chain_begin(nxt, steps, graph=graph)
    e1.record(stream)
    toks = m.chain_end(steps)
    wall = time.perf_counter() - t0
    dev_ms = e0.elapsed_time(e1)
    same = True
    # The greedy trajectory of a random-init model can sit on one repeated token, so equal tokens say little:
    # the last step's logits are compared across the ranks (and, by the caller, with the one-GPU run).
    logits = m.logits()
    logits_diff_ranks = 0.0
    row_lo, row_hi = m.logit_rows()
    choice = "all logits gathered on every rank, then the choice"
    if dist is not None and world > 1:
        dev_ms = float(reduce(torch.tensor([dev_ms], dtype=torch.float64), dist.ReduceOp.MAX).item())
        mine = torch.tensor([int(x) for x in toks], dtype=torch.int64)
        same = bool((reduce(mine.clone(), dist.ReduceOp.MIN) == reduce(mine.clone(), dist.ReduceOp.MAX)).all())
        if (row_lo, row_hi) != (0, cfg["V"]):
            # Only the ranks' (value, index) keys travelled: every rank holds its own rows of the last logits. They are
            # put together here, after the timed region, so that the whole vector can be compared with the one-GPU run.
            choice = "each rank chooses over its rows of the head; only the ranks' (value, index) keys are exchanged"
            whole = torch.zeros(cfg["V"], dtype=torch.float32)
            whole[row_lo:row_hi] = torch.from_numpy(logits[row_lo:row_hi].copy())
            logits = reduce(whole, dist.ReduceOp.SUM).numpy()
        else:
            llo = reduce(torch.from_numpy(logits.copy()), dist.ReduceOp.MIN)
            lhi = reduce(torch.from_numpy(logits.copy()), dist.ReduceOp.MAX)
            logits_diff_ranks = float((lhi - llo).max())
    tr = summarize_trace(L, 5 * cfg["L"] + 1) if trace and rank == 0 else None
    wbytes = chain_weight_bytes(cfg)
    rec = {"n_gpus": world,
           "sharding": "none" if world == 1 else "FFN and LM-head rows over ranks, " +
           ("rows stored into the peers' buffers by the GEMVs, flags" if gather == "peer" else "NCCL all-gather after each"),
           "tokens_equal_on_all_ranks": same,
           "lm_head_choice": choice if world > 1 else "one GPU",
           "lane": "CUDA graph per token" if graph else "host call per op",
           "decode_tok_per_s": round(steps / (dev_ms * 1e-3), 1), "ms_per_token": round(dev_ms / steps, 4),
           "wall_tok_per_s": round(steps / wall, 1),
           "prompt_tok_per_s": round(prompt_n / t_prompt, 1),
           "prompt_path": "layer stack" if prefill_gpu_ms is not None else "decode lane, token by token",
           "prompt_gpu_ms": None if prefill_gpu_ms is None else round(prefill_gpu_ms, 3),
           "prompt_tok_per_s_gpu": None if not prefill_gpu_ms else round(prompt_n / (prefill_gpu_ms * 1e-3), 1),
           "weight_bytes_per_token": wbytes,
           "weight_GBps": round(wbytes * steps / (dev_ms * 1e-3) / 1e9, 1),
           "kernels_encoded_per_chain_call": int(L.tm_cuda_launch_count()) - launches0,
           "first_tokens": [int(t) for t in toks[:8]], "distinct_tokens": len({int(t) for t in toks}),
           "last_logits_sha256": hashlib.sha256(logits.tobytes()).hexdigest()[:16],
           "last_logits_max_abs": float(np.abs(logits).max()),
           "last_logits_max_abs_diff_across_ranks": logits_diff_ranks,
           "trace": tr, "logits": logits}
    m.close()
    return rec


def run_chain(args, L, torch, rank: int = 0, world: int = 1) -> None:
    """Greedy decode chain of a random-init model: `--prompt` tokens fed one by one, then `--steps` chosen on the GPU.
    Under torch.distributed.run (world > 1) the FFN and LM-head rows are sharded over the ranks."""
    import time

    from . import chain
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("gloo")
        chain.init_comm(L, rank, world)
        if args.gather == "peer":
            chain.init_peer(L, rank, world, chain.peer_arena_bytes(cfg_for(args)))
    cfg = cfg_for(args)
    t0 = time.perf_counter()
    w = synth.make_llama(cfg, seed=5)
    t_gen = time.perf_counter() - t0
    rec = measure_chain(L, torch, cfg, w, args.prompt, args.steps, rank, world, args.gather, dist, not args.no_graph, args.trace,
                        args.prefill)
    logits = rec.pop("logits")
    if args.dump_logits and rank == 0:
        np.save(args.dump_logits, logits)
    if rank == 0:
        print(json.dumps(dict({"op": "chain", "model": args.model, "prompt": args.prompt, "steps": args.steps}, **rec,
                              model_build_s=round(t_gen, 1))), flush=True)
    if dist:
        dist.barrier()
        lib.check(L.tm_cuda_comm_destroy(), "tm_cuda_comm_destroy")
        lib.check(L.tm_cuda_peer_unmap(), "tm_cuda_peer_unmap")
        dist.barrier()
        lib.check(L.tm_cuda_peer_close(), "tm_cuda_peer_close")
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", choices=["gemv", "gemm", "dequant", "chain"], default="gemv")
    ap.add_argument("--model", choices=["llama3-8b", "tiny"], default="llama3-8b", help="architecture of --op chain")
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--gather", choices=["nccl", "peer"], default="peer", help="--op chain on several GPUs: how shards are gathered")
    ap.add_argument("--no-graph", action="store_true", help="--op chain: one host call per op instead of the graph lane")
    ap.add_argument("--prefill", choices=["feed", "stack"], default="feed",
                    help="--op chain: the prompt token by token through the decode lane, or as one batch through the layer stack")
    ap.add_argument("--dump-logits", default="", help="--op chain: rank 0 saves the last step's logits to this .npy file")
    ap.add_argument("--trace", action="store_true", help="--op chain with TM_CUDA_TRACE=1: add the per-kernel timeline summary")
    ap.add_argument("--dtype", default="Q8_0", choices=sorted(NAMES))
    ap.add_argument("--m", type=int, default=2000)
    ap.add_argument("--n", type=int, default=32000)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--copies", type=int, default=1, help="distinct weight copies to rotate over")
    ap.add_argument("--graph", action="store_true", help="capture the timed launches in one CUDA graph (no host launch cost)")
    args = ap.parse_args()

    import os

    import torch
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    dev = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(dev)
    L = lib.load()
    lib.check(L.tm_cuda_init(dev), "tm_cuda_init")
    if args.op == "chain":
        run_chain(args, L, torch, rank, world)
        return
    dt = NAMES[args.dtype]
    n, k, m = args.n, args.k, args.m
    W = synth.make_weights(dt, n, k, seed=1).reshape(-1)
    Ws = []
    for _ in range(args.copies):
        t = torch.zeros(W.size + 32, dtype=torch.uint8, device="cuda")
        t[: W.size] = torch.from_numpy(W).cuda()
        Ws.append(t)
    stream = torch.cuda.Stream()
    sp = C.c_void_p(stream.cuda_stream)
    vp = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731

    if args.op == "gemv":
        x = torch.from_numpy(synth.make_activations(k, 1)).cuda()
        y = torch.zeros(n, dtype=torch.float32, device="cuda")
        run = lambda i: lib.check(L.tm_cuda_gemv_q_dev(vp(x), vp(Ws[i % len(Ws)]), vp(y), n, k, dt, sp), "gemv")  # noqa: E731
        work, unit = synth.gemv_bytes(dt, n, k) / 1e9, "GB/s"
    elif args.op == "dequant":
        out = torch.zeros(n * k, dtype=torch.float32, device="cuda")
        run = lambda i: lib.check(L.tm_cuda_dequant_dev(vp(Ws[i % len(Ws)]), vp(out), n, k, dt, sp), "dequant")  # noqa: E731
        work, unit = (synth.weight_bytes(dt, n, k) + 4.0 * n * k) / 1e9, "GB/s"
    else:
        A = torch.from_numpy(synth.make_activations((m, k), 4)).cuda()
        Cm = torch.zeros((m, n), dtype=torch.float32, device="cuda")
        need = L.tm_cuda_sgemm_q_workspace(m, n, k, dt)
        ws = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
        base = C.c_void_p((ws.data_ptr() + 255) // 256 * 256)
        run = lambda i: lib.check(L.tm_cuda_sgemm_q_dev(vp(A), vp(Ws[i % len(Ws)]), vp(Cm), m, n, k, dt, base, need, sp), "gemm")  # noqa: E731
        work, unit = 2.0 * m * n * k / 1e12, "TFLOP/s"

    with torch.cuda.stream(stream):
        for i in range(args.warmup):
            run(i)
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if args.graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i in range(args.reps):
                    run(i)
            g.replay()
            stream.synchronize()
            e0.record(stream)
            g.replay()
            e1.record(stream)
        else:
            e0.record(stream)
            for i in range(args.reps):
                run(i)
            e1.record(stream)
        stream.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.reps
    lib.check(L.tm_cuda_tok_flush(), "device status")
    if args.trace and args.op == "gemv":
        # CTA 0's timeline of the last `reps` launches (TM_CUDA_TRACE=1): phases and the gap to the previous launch's end
        buf = (C.c_ulonglong * (6 * 8192))()
        nrec = int(L.tm_cuda_trace_read(buf, 8192))
        if nrec:
            a = np.frombuffer(buf, dtype=np.uint64)[: nrec * 6].reshape(nrec, 6).astype(np.int64)
            a = a[np.argsort(a[:, 0])][-args.reps:]
            gap = (a[1:, 0] - a[:-1, 3]) / 1e3
            print(json.dumps({"trace_us": {"wait": round(float((a[:, 1] - a[:, 0]).mean()) / 1e3, 2),
                                           "x": round(float((a[:, 2] - a[:, 1]).mean()) / 1e3, 2),
                                           "rows": round(float((a[:, 3] - a[:, 2]).mean()) / 1e3, 2),
                                           "start_to_end": round(float((a[:, 3] - a[:, 0]).mean()) / 1e3, 2),
                                           "end_to_next_start": round(float(gap.mean()), 2) if gap.size else None,
                                           "start_to_next_start": round(float((a[1:, 0] - a[:-1, 0]).mean()) / 1e3, 2) if gap.size else None}}))
    print(json.dumps({"op": args.op, "dtype": args.dtype, "m": m if args.op == "gemm" else None, "n": n, "k": k,
                      "us_per_launch": round(us, 3), "rate": round(work / (us * 1e-6), 2), "unit": unit,
                      "launches": int(L.tm_cuda_launch_count())}))


if __name__ == "__main__":
    main()
