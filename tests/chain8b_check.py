"""Decode-chain parity at the Llama-3-8B geometry (BASELINE config 5), run as a child process.

    python tests/chain8b_check.py [--positions 8] [--start 512] [--layers 0,15,31]

The GPU K/V cache precision is fixed when the library starts (TM_CUDA_KV_HALF), so the pytest wrapper
(tests/test_gpu_chain8b.py) runs this script once per mode and asserts on the JSON line it prints.

What is compared (CPU side: oracle/tm_oracle.c `tmo_chain_step`, the restated reference block loop):
  1. Teacher-forced logits. Both K/V caches are preloaded with the same random rows for positions
     [0, start), then `positions` tokens are fed at positions start, start+1, ... to the CPU chain and to
     the GPU per-op lane (the reference's encode order); bar 1e-3 * max|logit| (the reference's own
     GPU-vs-CPU bar with fp32 glue, test_llama_gpu_stack.cpp:10-14). With the half K/V cache the CPU side
     rounds K/V rows to fp16 as they are written, as the GPU cache does, and the same bar applies.
  2. One more position through the captured graph lane (fused norms / SiLU / residuals, one-launch
     attention) against the CPU chain: same bar.
  3. Op-boundary vectors of the last layer on the GPU (q after rope, v, attention output, SiLU*up,
     residual stream) against the CPU taps: 1e-3 * max|ref| (glue bar).
  4. Per projection, at the sampled layers: the GPU GEMV on the CPU chain's own input vector for q|k|v, o,
     gate, up, down and the Q6_K head against the fp64 dot of the dequantized row:
     |y - y64| <= 1e-3 * sum|w x| per output (the bar of the single-matrix configs).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import binding  # noqa: E402
from tensormark_b200 import chain, lib, synth  # noqa: E402

SLOT_X, SLOT_QKV, SLOT_AO, SLOT_GU, SLOT_KC, SLOT_VC = 0, 2, 3, 6, 100, 200


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--positions", type=int, default=8)
    ap.add_argument("--start", type=int, default=512)
    ap.add_argument("--layers", default="0,15,31")
    ap.add_argument("--model", default="llama3-8b", choices=["llama3-8b", "tiny"])
    args = ap.parse_args()
    kv_half = os.environ.get("TM_CUDA_KV_HALF", "1") != "0"

    cfg = dict(synth.LLAMA3_8B if args.model == "llama3-8b" else synth.TINY_CHAIN)
    start = args.start if args.model == "llama3-8b" else min(args.start, 40)
    Lh, D, H, KVH, dh, F, V, ctx = (cfg[k] for k in ("L", "D", "H", "KVH", "dh", "F", "V", "ctx"))
    QD, KVD = H * dh, KVH * dh
    layers = [min(int(s), Lh - 1) for s in args.layers.split(",")]
    layers = sorted(set(layers) | {Lh - 1})
    npos = max(args.positions, len(layers))
    assert start + npos + 1 <= ctx

    L = lib.load()
    lib.check(L.tm_cuda_init(0), "tm_cuda_init")
    orc = binding.oracle()
    threads = os.cpu_count() or 1
    t0 = time.perf_counter()
    w = synth.make_llama(cfg, seed=5)
    build_s = time.perf_counter() - t0

    cpu = binding.ChainModel(orc, cfg, w, kv_half=kv_half, threads=threads)
    gpu = chain.Chain(cfg, w)
    toks = synth.make_tokens(npos + 1, V, seed=5)

    # ---- the same history on both sides: random K/V rows for positions [0, start)
    gpu.forward(int(toks[0]))                      # sizes the slots and the caches; its row is overwritten below
    g = synth.rng_for(5, 11)
    for l in range(Lh):
        for name, arr, slot in (("k", cpu.kc, SLOT_KC), ("v", cpu.vc, SLOT_VC)):
            rows = g.standard_normal((KVH, start, dh), dtype=np.float32)
            if kv_half:
                rows = rows.astype(np.float16).astype(np.float32)
            arr[l, :, :start, :] = rows
            for h in range(KVH):
                blk = np.ascontiguousarray(rows[h])
                lib.check(L.tm_cuda_tok_kv_upload(slot + l, (h * ctx) * dh, blk.ctypes.data, blk.size), "kv_upload")
    gpu.seen = start

    out = {"model": args.model, "kv_half": kv_half, "start": start, "positions": npos, "layers": layers,
           "model_build_s": round(build_s, 1), "cpu_threads": threads}
    tap_at = {npos - len(layers) + i: l for i, l in enumerate(layers)}      # step index -> tapped layer
    taps = {}
    worst_logit, logit_bar_ok = 0.0, True
    cpu_s = 0.0
    last_gpu_boundary = None
    for i in range(npos):
        pos = start + i
        t0 = time.perf_counter()
        if i in tap_at:
            want, tp = cpu.step(int(toks[i]), pos, tap_layer=tap_at[i])
            taps[tap_at[i]] = tp
        else:
            want = cpu.step(int(toks[i]), pos)
        cpu_s += time.perf_counter() - t0
        got = gpu.forward(int(toks[i]))
        assert gpu.seen == pos + 1
        scale = max(1.0, float(np.abs(want).max()))
        err = float(np.abs(got - want).max()) / scale
        worst_logit = max(worst_logit, err)
        logit_bar_ok = logit_bar_ok and err <= 1e-3 and bool(np.isfinite(got).all())
        if i in tap_at and tap_at[i] == Lh - 1:
            # the per-op lane leaves the last layer's vectors in its slots
            def slot(s, off, n):
                a = np.empty(n, np.float32)
                lib.check(L.tm_cuda_tok_download(s, off * 4, a.ctypes.data, n * 4), "download")
                return a
            last_gpu_boundary = dict(q=slot(SLOT_QKV, 0, QD), v=slot(SLOT_QKV, QD + KVD, KVD), ao=slot(SLOT_AO, 0, QD),
                                     act=slot(SLOT_GU, 0, F), x_out=slot(SLOT_X, 0, D))
    out["logits_rel_err_max"] = worst_logit
    out["logits_ok"] = logit_bar_ok
    out["cpu_s_per_step"] = round(cpu_s / npos, 3)

    # ---- one more position through the graph lane
    pos = start + npos
    want = cpu.step(int(toks[npos]), pos)
    g_tokens, g_logits = gpu.greedy(int(toks[npos]), 1, graph=True)
    scale = max(1.0, float(np.abs(want).max()))
    out["graph_lane_rel_err"] = float(np.abs(g_logits - want).max()) / scale
    out["graph_lane_ok"] = out["graph_lane_rel_err"] <= 1e-3
    top2 = np.sort(want)[-2:]
    out["graph_lane_token_ok"] = bool(int(g_tokens[0]) == int(np.argmax(want)) or (top2[1] - top2[0]) <= 1e-3 * scale)

    # ---- op-boundary vectors of the last layer
    tp = taps[Lh - 1]
    o = 0
    ref = {}
    for name, n in (("h", D), ("qkv", QD + 2 * KVD), ("ao", QD), ("x_attn", D), ("h2", D), ("act", F), ("x_out", D)):
        ref[name] = tp[o:o + n]; o += n
    pairs = {"q": ref["qkv"][:QD], "v": ref["qkv"][QD + KVD:], "ao": ref["ao"], "act": ref["act"], "x_out": ref["x_out"]}
    glue = {k: float(np.abs(last_gpu_boundary[k] - v).max() / max(1e-30, float(np.abs(v).max()))) for k, v in pairs.items()}
    out["glue_rel_err"] = glue
    out["glue_ok"] = all(e <= 1e-3 for e in glue.values())
    gpu.close()                                   # also drops the lane's weight registrations

    # ---- per projection on the CPU chain's own inputs
    proj_worst, proj_ok = {}, True

    def check(tag, dt, W, x, n, k):
        nonlocal proj_ok
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty(n, np.float32)
        lib.check(L.tm_cuda_gemv_q(x.ctypes.data, W.ctypes.data, y.ctypes.data, n, k, dt), "tm_cuda_gemv_q")
        y64, yabs = orc.gemv_f64(dt, W, x, n, k)
        r = float((np.abs(y - y64) / np.maximum(yabs, 1e-30)).max())
        proj_worst[tag] = max(proj_worst.get(tag, 0.0), r)
        proj_ok = proj_ok and r <= 1e-3

    for l in layers:
        tp = taps[l]
        h, ao, h2, act = tp[:D], tp[D + QD + 2 * KVD: D + 2 * QD + 2 * KVD], None, None
        o = D + QD + 2 * KVD + QD + D
        h2, act = tp[o:o + D], tp[o + D:o + D + F]
        dt = cfg["dt_proj"]
        check("q", dt, w[f"l{l}.q"], h, QD, D)
        check("k", dt, w[f"l{l}.k"], h, KVD, D)
        check("v", dt, w[f"l{l}.v"], h, KVD, D)
        check("o", dt, w[f"l{l}.o"], ao, D, QD)
        check("gate", dt, w[f"l{l}.gate"], h2, F, D)
        check("up", dt, w[f"l{l}.up"], h2, F, D)
        check("down", dt, w[f"l{l}.down"], act, D, F)
        L.tm_cuda_release_weights()
    xf = orc.rmsnorm(ref["x_out"], w["rmsf"], cfg["eps"])
    check("head", cfg["dt_head"], w["head"], xf, V, D)
    L.tm_cuda_release_weights()
    out["proj_rel_err_max"] = proj_worst
    out["proj_ok"] = proj_ok
    out["status_ok"] = bool(L.tm_cuda_tok_flush())
    out["ok"] = bool(out["logits_ok"] and out["graph_lane_ok"] and out["graph_lane_token_ok"] and out["glue_ok"]
                     and out["proj_ok"] and out["status_ok"])
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
