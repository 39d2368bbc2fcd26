"""The reference arm of bench.py runs on the host cores alone: its one JSON line must keep the contract's keys
whatever the workload, and ranks other than 0 must stay silent."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(extra, env=None):
    e = dict(os.environ)
    e.pop("RANK", None)
    e.pop("WORLD_SIZE", None)
    e.update(env or {})
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2",
                          "--warmup", "1"] + extra, capture_output=True, text=True, env=e, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    return res.stdout


@pytest.mark.parametrize("workload,dtype", [("headline", "i8"), ("fp8", "f8e4m3"), ("fp32", "tf32")])
def test_reference_arm_line(workload, dtype):
    out = _run(["--workload", workload, "--sparsity", "0.98"])          # few tiles: a pass takes milliseconds
    lines = [ln for ln in out.splitlines() if ln.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "impl", "cpu_baseline", "e2e", "gpu_launches"):
        assert key in d, key
    assert d["impl"] == "reference" and d["metric"] == "block_sparse_spmm_tops_nonzero_tiles" and d["unit"] == "TOPS"
    assert d["dtype"] == dtype and d["data"] == "synthetic" and d["higher_is_better"] is True and d["gpu_launches"] == 0
    assert d["value"] > 0 and d["steps"] >= 1 and "workload" in d["config"] and "model" not in d["config"]
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_other_ranks_print_nothing():
    assert _run(["--workload", "headline", "--sparsity", "0.98", "--gpus", "2"], {"RANK": "1", "WORLD_SIZE": "2"}).strip() == ""
