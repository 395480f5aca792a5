"""The benchmark's JSON contract: the line `bench.py` prints carries the keys the contract names, on a
small case (GPU), and the host-core arm prints its line without a GPU."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE = ["metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
        "vs_baseline", "dtype", "data", "config"]


def _run(args, timeout):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py")] + args, cwd=ROOT, capture_output=True,
                         text=True, timeout=timeout)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.strip().splitlines() if ln.startswith("{")]
    assert len(lines) == 1, out.stdout[-2000:]
    return json.loads(lines[0])


def test_reference_arm_line_on_host_cores():
    line = _run(["--impl", "reference", "--steps", "1", "--warmup", "1"], timeout=600)
    for k in BASE:
        assert k in line, k
    assert line["impl"] == "reference" and line["value"] > 0 and line["higher_is_better"] is True
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in line["config"]


@pytest.mark.gpu
def test_bench_line_on_a_small_case(cuda_device):
    line = _run(["--batch", "2", "--steps", "3", "--warmup", "3", "--no-cpu", "--no-sustained", "--no-config5"], timeout=900)
    for k in BASE:
        assert k in line, k
    assert line["n_gpus"] == 1 and line["steps"] == 3 and line["value"] > 0 and line["gpu_launches"] > 0
    assert line["metric"] == "attn_fwd_bwd_tflops_windowed_causal" and line["unit"] == "TFLOP/s"
    r = line["roofline"]
    for k in ("bound", "achieved", "peak", "unit", "frac", "traffic", "kernels"):
        assert k in r, k
    assert 0 < r["frac"] < 1.2
    for name in ("attn_fwd", "attn_bwd_dq", "attn_bwd_dkv", "rope_pair_bf16_128", "linear_fwd"):
        assert name in r["kernels"], name
    e = line["e2e"]
    assert e["value"] > 0 and e["h2d_bytes_per_step"] > 0 and e["d2h_bytes_per_step"] > 0
    assert "sm_mhz" in line["clocks"] and "workload" in line["config"]
