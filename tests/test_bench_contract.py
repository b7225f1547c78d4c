"""The JSON line of ``bench.py``: keys and invariants that the harness around it reads.

Only the reference arm can run without a GPU (it times the CPU restatement of the unfused
decomposition, autoparallel/asynctp_ops.py:648-666 and :1124-1141, on host cores); the product
arm must refuse to run without one instead of falling back to anything.
"""
from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent

BASE_KEYS = {
    "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
    "scaling", "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches",
}


def _run(*args: str, timeout: int = 600) -> subprocess.CompletedProcess:
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], cwd=ROOT, capture_output=True, text=True, timeout=timeout)


def _json_lines(out: str) -> list[dict]:
    return [json.loads(l) for l in out.splitlines() if l.startswith("{")]


def test_reference_arm_prints_one_contract_line():
    res = _run("--impl", "reference", "--steps", "1", "--warmup", "1")
    assert res.returncode == 0, res.stderr[-2000:]
    lines = _json_lines(res.stdout)
    assert len(lines) == 1, res.stdout
    d = lines[0]
    assert d["impl"] == "reference"
    assert BASE_KEYS <= set(d), BASE_KEYS - set(d)
    assert d["n_gpus"] == 1 and d["steps"] == 1 and d["warmup"] == 1
    assert d["higher_is_better"] is True and d["scaling"] == "weak" and d["data"] == "synthetic"
    assert d["vs_baseline"] is None
    assert d["value"] > 0 and d["ms_per_step"] > 0
    assert "workload" in d["config"] and "model" not in d["config"]
    # the CPU arm launches no kernels and moves nothing over PCIe
    assert d["gpu_launches"] == 0
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]


def test_reference_arm_metric_matches_workload_flops():
    """value = flops of the sampled tokens / time: recompute it from the line's own fields."""
    res = _run("--impl", "reference", "--steps", "1", "--warmup", "1")
    d = _json_lines(res.stdout)[0]
    c = d["config"]
    sample_tokens = int(d["cpu_baseline"]["sample"].split()[0])
    flops = 2.0 * sample_tokens * c["hidden"] * c["ffn_per_rank"] * 3  # w1, w3 and w2
    assert d["unit"] == "TFLOP/s"
    assert d["value"] == pytest.approx(flops / (d["ms_per_step"] * 1e-3) / 1e12, rel=1e-6)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour of a box without a GPU")
def test_product_arm_refuses_to_run_without_a_gpu():
    res = _run("--steps", "1", "--warmup", "1", "--no-cpu-baseline", timeout=300)
    assert res.returncode != 0
    assert _json_lines(res.stdout) == []
