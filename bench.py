#!/usr/bin/env python
"""Benchmark of the quantized-weight matmul path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the decode GEMV over the Q8_0 + Q4_1 sweep at the
TinyLlama-1.1B projection shapes (2048x2048, 256x2048, 5632x2048, 2048x5632,
32000x2048; ten GEMVs, 160 MB of blocks). The metric is algorithmic bytes per
second: sum over the sweep of (block payload + 4*in + 4*out) divided by device time.

  value      device-resident: weights, x and y live in HBM; the ten launches of a step
             are captured in one CUDA graph and the graph is replayed K times between
             two CUDA events on the launching stream. The weights rotate over three
             copies per matrix (480 MB), so a buffer is reused only after more than
             twice the 126 MB L2 has been streamed.
  e2e        the same sweep through the host-pointer C ABI (tm_cuda_gemv_q): x comes
             from pinned host memory and y goes back to the host inside the timed
             region, one blocking call per GEMV. Weights are cached on the device on
             first use, which is the contract of the entry point being replaced.
             At N > 1 every rank does this on its own GPU; the slowest rank's time counts.
  roofline   the GEMV kernel against the measured HBM copy bandwidth.
  cpu_baseline  the CPU restatement of the reference's dot path on the host cores.

With --gpus N > 1 (launched by torch.distributed.run, one rank per GPU) every rank runs
the whole sweep on its own activation vectors: N independent decode streams, no
collective on the data path, per-GPU work fixed ("weak" scaling). These projection
shapes are small enough that one GPU finishes each GEMV in 2-12 us, which is less than
one all-gather costs, so they stay whole on a GPU. --shard selects the other layout for
comparison: matrices of >= 4096 rows split by output rows over the ranks and their
outputs all-gathered with NCCL; total work is then fixed ("strong" scaling).
"""
from __future__ import annotations

import argparse
import datetime
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from tensormark_b200 import shard, synth  # noqa: E402

SWEEP = [(dt, shape) for dt in (synth.Q8_0, synth.Q4_1) for shape in synth.TINYLLAMA_SHAPES]
SEEDS = {synth.Q8_0: 1, synth.Q4_1: 2}
COPIES = 3
WORKLOAD = "Q8_0+Q4_1 decode GEMV sweep, TinyLlama-1.1B projection shapes (BASELINE config 2)"


def note(rank: int, msg: str) -> None:
    """Progress marker on stderr (TM_BENCH_VERBOSE=1): which phase each rank has reached."""
    if os.environ.get("TM_BENCH_VERBOSE") == "1":
        print(f"[bench rank {rank}] {msg}", file=sys.stderr, flush=True)


def sweep_bytes() -> int:
    return sum(synth.gemv_bytes(dt, n, k) for dt, (n, k) in SWEEP)


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def recorded_traffic():
    """DRAM bytes per launch of the dominant kernel, taken from the committed ncu summary (or None)."""
    path = os.path.join(ROOT, "profiles", "gemv_traffic.json")
    if os.path.exists(path):
        try:
            return json.load(open(path))
        except Exception:
            return None
    return None


def measured_tensor_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            return float(d["bf16_tflops"]), float(d["bf16_tflops_sustained"]), "measured"
        except Exception:
            pass
    return 1590.0, 1400.0, "fallback"


def _half(b: np.ndarray) -> np.ndarray:
    """[..., 2] little-endian bytes -> fp32 value of the IEEE half."""
    return np.ascontiguousarray(b).view(np.float16)[..., 0].astype(np.float32)


def dequant_rows_numpy(dt: int, rows: np.ndarray) -> np.ndarray:
    """fp32 weights of whole rows of blocks (uint8 [r, row_bytes]), written from the block layouts
    (tensormark/quant.h:36-46, 215-220, 239-245) in numpy, each product rounded to fp32 as the scalar dequantizers do.
    Used only to spot-check what the timed region computed."""
    r = rows.shape[0]
    if dt == synth.Q8_0:
        b = rows.reshape(r, -1, 34)
        return (b[:, :, 2:].view(np.int8).astype(np.float32) * _half(b[:, :, 0:2])[..., None]).reshape(r, -1)
    if dt == synth.Q4_0:
        b = rows.reshape(r, -1, 18)
        q = np.stack([b[:, :, 2:] & 15, b[:, :, 2:] >> 4], axis=-1).reshape(r, -1, 32).astype(np.float32) - 8.0
        return (q * _half(b[:, :, 0:2])[..., None]).reshape(r, -1)
    if dt == synth.Q4_1:
        b = rows.reshape(r, -1, 20)
        q = np.concatenate([b[:, :, 4:] & 15, b[:, :, 4:] >> 4], axis=-1).astype(np.float32)
        return (q * _half(b[:, :, 0:2])[..., None] + _half(b[:, :, 2:4])[..., None]).reshape(r, -1)
    if dt == synth.Q6_K:
        b = rows.reshape(r, -1, 210)
        ql, qh, sc, d = b[..., 0:128], b[..., 128:192], b[..., 192:208].view(np.int8), _half(b[..., 208:210])
        out = np.empty(b.shape[:2] + (256,), np.float32)
        for h in range(2):
            for j in range(4):
                lo = ql[..., 64 * h + 32 * (j & 1): 64 * h + 32 * (j & 1) + 32]
                lo = (lo >> 4) if j >= 2 else (lo & 15)
                hi = (qh[..., 32 * h: 32 * h + 32] >> (2 * j)) & 3
                q = (lo | (hi << 4)).astype(np.float32) - 32.0
                s = np.repeat(sc[..., 8 * h + 2 * j: 8 * h + 2 * j + 2], 16, axis=-1).astype(np.float32)
                out[..., 128 * h + 32 * j: 128 * h + 32 * j + 32] = (d[..., None] * s) * q
        return out.reshape(r, -1)
    raise ValueError(dt)


def check_gemv_rows(dt: int, W: np.ndarray, x: np.ndarray, y: np.ndarray, nrows: int = 16, seed: int = 0):
    """Sampled outputs of a GEMV against fp64 dots of the dequantized rows: worst |y - y64| / sum|w x| (bar 1e-3)."""
    idx = np.unique(np.random.default_rng(seed).integers(0, W.shape[0], size=nrows))
    w = dequant_rows_numpy(dt, W[idx]).astype(np.float64)
    p = w * x.astype(np.float64)[None, :]
    return float((np.abs(y[idx] - p.sum(1)) / np.maximum(np.abs(p).sum(1), 1e-30)).max())


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._pump, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass

    def summary(self):
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- reference arm
def run_reference(args, rank: int):
    """The reference's CPU dot path (restated; its own header does not build on Linux) on all host threads.
    One step = one pass over the same sweep."""
    if rank != 0:
        return
    from oracle import binding
    orc = binding.oracle_fast()
    threads = os.cpu_count() or 1
    mats = [(dt, n, k, synth.make_weights(dt, n, k, SEEDS[dt]), synth.make_activations(k, SEEDS[dt])) for dt, (n, k) in SWEEP]

    def step():
        for dt, n, k, W, x in mats:
            orc.gemv(dt, W, x, n, k, threads=threads)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt_s = time.perf_counter() - t0
    val = sweep_bytes() * args.steps / dt_s / 1e9
    line = {
        "impl": "reference", "metric": "decode_gemv_algorithmic_bandwidth", "value": val, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt_s / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "where": "host CPU"},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": "the full sweep (10 GEMVs, 160 MB of blocks) per step, 64-row chunks over all host threads"},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- extra records of our arm
GEMM_SHAPES = [(synth.Q4_0, 5632, 2048), (synth.Q4_0, 2048, 5632), (synth.Q6_K, 32000, 2048)]
GEMM_M = 2000


def gemm_record(L, lib, torch, calls: int = 20):
    """BASELINE config 4: X (2000 tokens, fp32) against the three quantized matrices through tm_cuda_sgemm_q_dev,
    device-resident, CUDA events around `calls` back-to-back calls (each call includes its operand preparation).
    Three copies of A, W and C are rotated so that no call finds its operands in L2."""
    burst, sustained, kind = measured_tensor_peaks()
    stream = torch.cuda.Stream()
    sp = C.c_void_p(stream.cuda_stream)
    vp = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    out = []
    for dt, n, k in GEMM_SHAPES:
        m = GEMM_M
        W = synth.make_weights(dt, n, k, seed=4)
        A = synth.make_activations((m, k), seed=4)
        Ws, As, Cs = [], [], []
        for _ in range(3):
            t = torch.zeros(W.size + 32, dtype=torch.uint8, device="cuda")
            t[: W.size] = torch.from_numpy(W.reshape(-1)).cuda()
            Ws.append(t)
            As.append(torch.from_numpy(A).cuda())
            Cs.append(torch.zeros((m, n), dtype=torch.float32, device="cuda"))
        need = int(L.tm_cuda_sgemm_q_workspace(m, n, k, dt))
        ws = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
        base = C.c_void_p((ws.data_ptr() + 255) // 256 * 256)
        before = int(L.tm_cuda_launch_count())
        with torch.cuda.stream(stream):
            def call(i):
                lib.check(L.tm_cuda_sgemm_q_dev(vp(As[i % 3]), vp(Ws[i % 3]), vp(Cs[i % 3]), m, n, k, dt, base, need, sp), "tm_cuda_sgemm_q_dev")
            for i in range(3):
                call(i)
            stream.synchronize()
            per_call = (int(L.tm_cuda_launch_count()) - before) // 3
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(calls):
                call(i)
            e1.record(stream)
            stream.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / calls
        tf = 2.0 * m * n * k / (us * 1e-6) / 1e12
        # spot check of what was just computed: 64 sampled outputs against fp64 dots of the dequantized rows
        rng = np.random.default_rng(n + k)
        mi, ni = rng.integers(0, m, size=64), rng.integers(0, n, size=64)
        w = dequant_rows_numpy(dt, W[ni]).astype(np.float64)
        pr = w * A[mi].astype(np.float64)
        got = Cs[(calls - 1) % 3][torch.from_numpy(mi).cuda(), torch.from_numpy(ni).cuda()].cpu().numpy()
        worst = float((np.abs(got - pr.sum(1)) / np.maximum(np.abs(pr).sum(1), 1e-30)).max())
        assert worst <= 1e-3, f"GEMM outputs are off: {worst:.3e} of sum|a w| (bar 1e-3)"
        out.append({"dtype": synth.DTYPE_NAMES[dt], "M": m, "N": n, "K": k, "us_per_call": round(us, 2), "TFLOPs": round(tf, 1),
                    "frac_of_burst": round(tf / burst, 3), "frac_of_sustained": round(tf / sustained, 3),
                    "launches_per_call": per_call, "worst_err_over_sum_abs": worst})
        del Ws, As, Cs, ws
        torch.cuda.empty_cache()
    return {"workload": "prefill GEMM, BASELINE config 4 (M=2000 tokens, fp32 in/out, fp16 operands on tcgen05, fp32 accumulate)",
            "calls_timed": calls, "peak_burst_TFLOPs": burst, "peak_sustained_TFLOPs": sustained, "peak_kind": kind,
            "l2": "three copies of A, W and C rotated (each call's operands come from HBM)", "shapes": out}


def sharded_chain_record(L, lib, torch, dist, rank: int, world: int, prompt_n: int = 512, steps: int = 128):
    """BASELINE config 5: the Llama-3-8B-shaped decode chain (random-init weights, Q4_0 projections, Q6_K head), a
    512-token prompt then 128 greedy steps chosen on the GPU. At N > 1 the FFN and LM-head rows are split over the ranks
    and gathered through peer memory by the GEMVs themselves; the same ranks then run the chain unsharded, which gives
    the one-GPU time the speed-up is quoted against and the logits the sharded result must reproduce."""
    from tensormark_b200 import chain, run_case
    cfg = dict(synth.LLAMA3_8B)
    cfg["ctx"] = max(cfg["ctx"], prompt_n + steps + 1)
    t0 = time.perf_counter()
    w = synth.make_llama(cfg, seed=5)
    build_s = time.perf_counter() - t0
    bound_ms = run_case.chain_weight_bytes(cfg) / (measured_peak()[0] * 1e9) * 1e3
    rec = {"workload": "decode chain, BASELINE config 5 (Llama-3-8B shapes, prompt %d, %d greedy steps)" % (prompt_n, steps),
           "model_build_s": round(build_s, 1), "streaming_bound_ms_per_token_1gpu": round(bound_ms, 4)}
    sh, got = None, None
    if world > 1:
        # the sharded run comes first: its gathered slots live in the peer arena, and a slot of the lane cannot change
        # from private to shared; closing the arena afterwards returns them to the lane
        chain.init_comm(L, rank, world)
        chain.init_peer(L, rank, world, chain.peer_arena_bytes(cfg))
        sh = run_case.measure_chain(L, torch, cfg, w, prompt_n, steps, rank, world, "peer", dist, prefill="stack")
        got = sh.pop("logits")
        sh.pop("trace", None)
        dist.barrier()
        lib.check(L.tm_cuda_comm_destroy(), "tm_cuda_comm_destroy")
        lib.check(L.tm_cuda_peer_unmap(), "tm_cuda_peer_unmap")
        dist.barrier()
        lib.check(L.tm_cuda_peer_close(), "tm_cuda_peer_close")
        dist.barrier()
    one = run_case.measure_chain(L, torch, cfg, w, prompt_n, steps, 0, 1, "peer", None, prefill="stack")
    ref_logits = one.pop("logits")
    one.pop("trace", None)
    rec["one_gpu"] = dict(one, frac_of_streaming_bound=round(bound_ms / one["ms_per_token"], 3))
    if sh is not None:
        one_ms = torch.tensor([one["ms_per_token"]], dtype=torch.float64, device="cuda")
        dist.all_reduce(one_ms, op=dist.ReduceOp.MAX)
        one_ms = float(one_ms.item())
        scale = max(1.0, float(np.abs(ref_logits).max()))
        ceiling = 1.0 / (0.173 + 0.827 / world)
        rec["sharded"] = dict(sh, gather="peer stores + counters inside the GEMVs",
                              one_gpu_ms_per_token_max_over_ranks=round(one_ms, 4),
                              speedup_over_one_gpu=round(one_ms / sh["ms_per_token"], 3),
                              bytes_only_ceiling=round(ceiling, 2),
                              last_logits_max_abs_diff_vs_one_gpu=float(np.abs(got - ref_logits).max()),
                              last_logits_rel_diff_vs_one_gpu=float(np.abs(got - ref_logits).max()) / scale)
    return rec


# --------------------------------------------------------------------------- our arm
def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist
    from tensormark_b200 import lib

    # Libraries (NCCL's version banner among them) write to stdout: keep fd 1 for the one JSON line.
    sys.stdout.flush()
    out_fd = os.dup(1)
    os.dup2(2, 1)

    torch.cuda.set_device(local_rank)
    L = lib.load()
    lib.check(L.tm_cuda_init(local_rank), "tm_cuda_init")
    if world > 1:
        # a collective that one rank never joins ends the run after five minutes, not after NCCL's default of ten
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=300))

    def vp(t):
        return C.c_void_p(t.data_ptr())

    shard_world = world if args.shard else 1
    # ---- resident inputs: every matrix (this rank's row shard of it with --shard), COPIES times
    mats = []
    for dt, (n, k) in SWEEP:
        sharded = shard.is_sharded(n, shard_world)
        W = synth.make_weights(dt, n, k, SEEDS[dt])
        lo, hi = shard.row_range(n, rank if sharded else 0, shard_world if sharded else 1)
        Wl = np.ascontiguousarray(W[lo:hi]).reshape(-1)
        copies = []
        for _ in range(COPIES):
            t = torch.zeros(Wl.size + 32, dtype=torch.uint8, device="cuda")
            t[: Wl.size] = torch.from_numpy(Wl).cuda()
            copies.append(t)
        x = torch.from_numpy(synth.make_activations(k, SEEDS[dt])).cuda()
        y = torch.zeros(n, dtype=torch.float32, device="cuda")
        ypart = torch.zeros(hi - lo, dtype=torch.float32, device="cuda") if sharded else None
        mats.append(dict(dt=dt, n=n, k=k, rows=hi - lo, sharded=sharded, W=copies, x=x, y=y, ypart=ypart, host=(W, lo, hi)))

    stream = torch.cuda.Stream()
    sp = C.c_void_p(stream.cuda_stream)
    note(rank, "inputs resident")

    def launch_step(copy: int):
        for m in mats:
            out = m["ypart"] if m["sharded"] else m["y"]
            ok = L.tm_cuda_gemv_q_dev(vp(m["x"]), vp(m["W"][copy]), vp(out), m["rows"], m["k"], m["dt"], sp)
            lib.check(ok, "tm_cuda_gemv_q_dev")
            if m["sharded"]:
                dist.all_gather_into_tensor(m["y"], m["ypart"])

    # ---- one graph per weight copy, so replays walk the copies round-robin
    graphs = []
    with torch.cuda.stream(stream):
        launch_step(0)
        stream.synchronize()
        note(rank, "first eager step done")
        before = L.tm_cuda_launch_count()
        launch_step(0)
        launches_per_step = int(L.tm_cuda_launch_count() - before)
        stream.synchronize()
        use_graph = os.environ.get("TM_BENCH_GRAPH", "1") != "0"
        if use_graph:
            try:
                for c in range(COPIES):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream):
                        launch_step(c)
                    graphs.append(g)
                note(rank, "graphs captured")
            except Exception as e:      # capture refused (e.g. a collective that cannot be captured): plain launches
                if rank == 0:
                    print(f"[bench] graph capture unavailable, using stream launches: {e}", file=sys.stderr)
                graphs = []
                torch.cuda.synchronize()

    def step(i: int):
        if graphs:
            graphs[i % COPIES].replay()
        else:
            launch_step(i % COPIES)

    # The timed steps go into as few graph launches as possible: one graph of up to 48 steps (walking the weight copies
    # step by step), replayed, plus one graph for the remainder. A graph launch per step would put a launch gap
    # between steps that a resident caller of the library does not have.
    big, rem, G = None, None, 0
    if graphs:
        try:
            with torch.cuda.stream(stream):
                G = min(args.steps, 48) // COPIES * COPIES
                if G:
                    big = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(big, stream=stream):
                        for i in range(G):
                            launch_step(i % COPIES)
                r = args.steps - (args.steps // G) * G if G else args.steps
                if r:
                    rem = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(rem, stream=stream):
                        for i in range(r):
                            launch_step(i % COPIES)
        except Exception as e:
            if rank == 0:
                print(f"[bench] multi-step graph unavailable, one graph launch per step: {e}", file=sys.stderr)
            big, rem, G = None, None, 0
            torch.cuda.synchronize()

    def timed_steps():
        if big is None and rem is None:
            for i in range(args.steps):
                step(args.warmup + i)
            return
        for _ in range(args.steps // G if G else 0):
            big.replay()
        if rem is not None:
            rem.replay()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(stream):
        for i in range(args.warmup):
            step(i)
        for g in (big, rem):                     # a graph's first launch uploads it: not in the timed region
            if g is not None:
                g.replay()
        barrier()
        note(rank, "warm-up done")
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as clk:
            ev0.record(stream)
            timed_steps()
            ev1.record(stream)
            barrier()
        ms = ev0.elapsed_time(ev1)
    note(rank, f"timed region done: {ms:.3f} ms")
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    total = sweep_bytes()
    replicas = 1 if args.shard else world
    value = replicas * total * args.steps / (ms * 1e-3) / 1e9

    # ---- correctness guard on what was just timed (cheap: sampled rows against numpy fp64)
    guard_worst = 0.0
    if rank == 0:
        for i, m in enumerate(mats):
            W, lo, hi = m["host"]
            yh = m["y"].cpu().numpy()
            assert np.isfinite(yh).all(), "non-finite GEMV output in the timed region"
            guard_worst = max(guard_worst, check_gemv_rows(m["dt"], W, m["x"].cpu().numpy(), yh, seed=i))
        assert guard_worst <= 1e-3, f"timed GEMV outputs are off: {guard_worst:.3e} of sum|w x| (bar 1e-3)"

    status_ok = bool(L.tm_cuda_tok_flush())          # harvests the device status word
    if not status_ok:
        raise RuntimeError("device status: " + lib.last_error())

    # ---- e2e: host-pointer C ABI, pinned x, y back to the host
    hx = {k: torch.from_numpy(synth.make_activations(k, 1)).pin_memory() for k in {m["k"] for m in mats}}
    hy = {m["n"]: torch.empty(m["n"], dtype=torch.float32).pin_memory() for m in mats}
    hW = [np.ascontiguousarray(m["host"][0]) for m in mats]

    def e2e_step():
        for m, W in zip(mats, hW):
            ok = L.tm_cuda_gemv_q(C.c_void_p(hx[m["k"]].data_ptr()), C.c_void_p(W.ctypes.data),
                                  C.c_void_p(hy[m["n"]].data_ptr()), m["n"], m["k"], m["dt"])
            lib.check(ok, "tm_cuda_gemv_q")

    # Every rank drives its own GPU through the host-pointer entry (independent replicas, as in the device-resident
    # sweep); the time is the slowest rank's wall clock between two barriers.
    for _ in range(max(3, args.warmup)):
        e2e_step()
    barrier()
    lb = L.tm_cuda_launch_count()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    es = time.perf_counter() - t0
    e2e_launches = int(L.tm_cuda_launch_count() - lb)
    if world > 1:
        t = torch.tensor([es], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        es = float(t.item())
    e2e = {"value": world * total * args.steps / es / 1e9, "unit": "GB/s",
           "h2d_bytes_per_step": world * sum(4 * m["k"] for m in mats), "d2h_bytes_per_step": world * sum(4 * m["n"] for m in mats),
           "ms_per_step": es / args.steps * 1e3, "gpu_launches": e2e_launches * world,
           "note": "blocking tm_cuda_gemv_q per GEMV on every rank's own GPU; weights cached on the device by (pointer, bytes) "
                   "as the replaced entry does; slowest rank's wall clock"}
    L.tm_cuda_release_weights()

    line = None
    if rank == 0:
        # ---- per-shape device numbers (each GEMV alone, rotating its copies; N=1 only)
        per_shape = []
        if world == 1:
            with torch.cuda.stream(stream):
                for m in mats:
                    reps = 24                                     # launches per graph, walking the copies
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream):
                        for r in range(reps):
                            L.tm_cuda_gemv_q_dev(vp(m["x"]), vp(m["W"][r % COPIES]), vp(m["y"]), m["n"], m["k"], m["dt"], sp)
                    for _ in range(3):
                        g.replay()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    nrep = 20
                    e0.record(stream)
                    for _ in range(nrep):
                        g.replay()
                    e1.record(stream)
                    stream.synchronize()
                    us = e0.elapsed_time(e1) * 1e3 / (reps * nrep)
                    b = synth.gemv_bytes(m["dt"], m["n"], m["k"])
                    per_shape.append({"dtype": synth.DTYPE_NAMES[m["dt"]], "shape": [m["n"], m["k"]], "us": round(us, 3),
                                      "GBps": round(b / us / 1e3, 1), "frac": round(b / us / 1e3 / measured_peak()[0], 3),
                                      "l2_resident": 3 * b < 126e6,
                                      "note": "24 launches per CUDA graph over 3 weight copies; a matrix whose 3 copies fit the "
                                              "126 MB L2 is served from L2, not HBM"})
                    del g

        # ---- CPU baseline (bounded sample, N=1 only)
        cpu = None
        if world == 1 and not args.no_cpu:
            from oracle import binding
            orc = binding.oracle_fast()
            threads = os.cpu_count() or 1
            t0 = time.perf_counter()
            reps = 0
            while reps < 1 or (time.perf_counter() - t0 < 10.0 and reps < 8):
                for m, W in zip(mats, hW):
                    orc.gemv(m["dt"], W, hx[m["k"]].numpy(), m["n"], m["k"], threads=threads)
                reps += 1
            cs = time.perf_counter() - t0
            cpu = {"value": total * reps / cs / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                   "sample": f"{reps} pass(es) over the full sweep (10 GEMVs, 160 MB of blocks), scalar dot path restated from the "
                             "reference, 64-row chunks over all host threads, gcc -O3 -march=native, no BLAS"}

        peak, peak_kind = measured_peak()
        traffic = recorded_traffic()
        clocks = clk.summary()
        line = {
            "metric": "decode_gemv_algorithmic_bandwidth", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong" if args.shard else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "gemvs_per_step": len(SWEEP), "bytes_per_step": total * replicas,
                       "l2": f"weights rotate over {COPIES} copies per matrix ({COPIES * 160} MB), more than 2x the 126 MB L2 between reuses",
                       "launch": (f"CUDA graphs of up to {G} steps" if big is not None or rem is not None else
                                  "one CUDA graph per step" if graphs else "stream launches"),
                       "sharding": ("single GPU" if world == 1 else
                                    "rows over ranks + NCCL all-gather for matrices with >= 4096 rows" if args.shard else
                                    "none: one independent sweep per GPU, no data-path collective")},
            "roofline": {"bound": "hbm", "achieved": value / world, "peak": peak, "unit": "GB/s", "frac": value / world / peak,
                         "peak_kind": peak_kind + " STREAM-style copy",
                         "traffic": (traffic or {}).get("dram_bytes_per_launch"),
                         "traffic_note": (traffic or {}).get("note"),
                         "kernel": "gemv_stream", "per_gpu": world > 1},
            "cpu_baseline": cpu,
            "e2e": e2e,
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "per_shape": per_shape,
            "guard": {"what": "16 sampled rows of every timed GEMV output against numpy fp64 dots of the dequantized rows",
                      "worst_err_over_sum_abs": guard_worst, "bar": 1e-3},
            "gemm": None,
            "sharded_chain": None,
        }

    # ---- the other two configs of the metric, in the same line. They run after the headline numbers exist, under a
    # watchdog: if one of them does not finish, the line is printed without it and the process ends.
    emitted = threading.Lock()

    def emit(final: bool):
        if not emitted.acquire(blocking=False):
            return
        if line is not None:
            os.write(out_fd, (json.dumps(line) + "\n").encode())
        if not final:
            os._exit(0)

    def give_up(what: str, limit_s: float):
        if line is not None and line.get(what) is None:
            line[what] = {"error": f"did not finish within {limit_s:.0f} s; left out"}
        emit(final=False)

    if rank == 0 and world == 1 and not args.no_gemm:
        dog = threading.Timer(120.0, give_up, ("gemm", 120.0)); dog.daemon = True; dog.start()
        try:
            line["gemm"] = gemm_record(L, lib, torch)
        except Exception as e:
            line["gemm"] = {"error": f"{type(e).__name__}: {e}"[:400]}
        dog.cancel()
    if not args.no_chain:                              # every rank takes part; rank 0 reports
        dog = threading.Timer(420.0, give_up, ("sharded_chain", 420.0)); dog.daemon = True; dog.start()
        try:
            rec = sharded_chain_record(L, lib, torch, dist, rank, world)
        except Exception as e:
            rec = {"error": f"{type(e).__name__}: {e}"[:400]}
        dog.cancel()
        if line is not None:
            line["sharded_chain"] = rec
    emit(final=True)
    if world > 1:
        # Graphs that captured collectives hold the communicator: release them before the group is
        # destroyed (destroying first waits for ever), and bound the teardown now that the line is out.
        graphs.clear()
        import gc
        gc.collect()
        torch.cuda.synchronize()
        guard = threading.Timer(30.0, lambda: os._exit(0))
        guard.daemon = True
        guard.start()
        note(rank, "teardown")
        dist.barrier()
        dist.destroy_process_group()
        guard.cancel()
        note(rank, "done")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-chain", action="store_true", help="skip the config-5 decode-chain record")
    ap.add_argument("--no-gemm", action="store_true", help="skip the config-4 prefill-GEMM record")
    ap.add_argument("--shard", action="store_true", help="N > 1: split large matrices by rows over the ranks and all-gather (strong scaling)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus:
        if args.gpus != 1 and world == 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run, one rank per GPU")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
