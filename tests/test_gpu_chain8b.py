"""Config-5 parity at its own geometry: Llama-3-8B shapes (32 layers, D 4096, 32/8 heads of 128, F 14336,
V 128256, Q4_0 projections, Q6_K head), positions 512.., both K/V cache precisions.

The checks themselves are in tests/chain8b_check.py (one child process per cache precision, because the
library reads TM_CUDA_KV_HALF once). Bars: logits 1e-3 * max|logit| teacher-forced against the CPU block
loop (tensormark/test_llama_gpu_stack.cpp:10-14), op-boundary vectors 1e-3, every projection
|y - y64| <= 1e-3 * sum|w x| on the CPU chain's own inputs."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(kv_half: str, model: str = "llama3-8b") -> dict:
    env = dict(os.environ, TM_CUDA_KV_HALF=kv_half)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "chain8b_check.py"), "--model", model],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert lines, r.stdout[-2000:]
    return json.loads(lines[-1])


@pytest.mark.gpu
@pytest.mark.parametrize("kv_half", ["1", "0"], ids=["half-kv", "fp32-kv"])
def test_llama3_8b_chain_matches_cpu_block_loop(torch_mod, kv_half):
    res = _run(kv_half)
    assert res["kv_half"] == (kv_half == "1")
    assert res["logits_ok"], res
    assert res["graph_lane_ok"] and res["graph_lane_token_ok"], res
    assert res["glue_ok"], res
    assert res["proj_ok"], res
    assert res["status_ok"] and res["ok"], res
