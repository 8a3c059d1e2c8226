"""The benchmark's command-line contract, as far as it can be exercised without a GPU: the
reference arm runs the CPU implementation and prints one JSON line with the agreed keys; the
product arm refuses to run without a CUDA device instead of falling back to anything."""
import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, env=None):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=300, env={**os.environ, **(env or {})})


def test_reference_arm_prints_the_contract_line():
    r = _run("--impl", "reference", "--steps", "2", "--warmup", "1", "--grid", "16")
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "spmv_fwd_bwd_effective_GBps" and line["unit"] == "GB/s"
    assert line["higher_is_better"] is True and line["vs_baseline"] is None and line["dtype"] == "f64"
    assert line["value"] > 0 and line["steps"] == 2
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] == 1
    assert line["cpu_baseline"]["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["config"]["workload"].startswith("poisson3d_7pt_16^3")


def test_reference_arm_other_ranks_exit_quietly():
    r = _run("--impl", "reference", "--steps", "2", "--warmup", "1", "--grid", "16", "--gpus", "2",
             env={"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"})
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_product_arm_needs_a_gpu():
    if torch.cuda.is_available():
        return                                   # on a GPU box the arm runs; covered by the bench itself
    r = _run("--steps", "1", "--warmup", "1", "--grid", "16", "--no-cpu-baseline")
    assert r.returncode != 0
    assert "CUDA" in (r.stderr + r.stdout)
