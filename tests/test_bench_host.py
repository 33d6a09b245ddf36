"""bench.py on a box without a GPU: the reference arm (the CPU restatement of the path, which needs no GPU) prints ONE
JSON line with the contract's keys, and the repo arm refuses to run without its CUDA library and a device instead of
falling back to anything."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, timeout=600):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], cwd=ROOT, capture_output=True, text=True,
                          timeout=timeout)


def test_reference_arm_prints_the_contract_line():
    r = _run("--impl", "reference", "--steps", "2", "--warmup", "1", "--tokens", "64")
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "dense_equiv_tflops_gated_ffn" and d["unit"] == "TFLOP/s"
    assert d["steps"] == 2 and d["warmup"] == 1 and d["n_gpus"] == 1 and d["higher_is_better"] is True
    assert d["config"]["tokens"] == 64 and d["config"]["hidden"] == 4096 and d["config"]["intermediate"] == 11008
    assert d["value"] > 0 and d["ms_per_step"] > 0
    # 6 * M * H * I flop per step
    assert abs(d["value"] - 6.0 * 64 * 4096 * 11008 / (d["ms_per_step"] * 1e-3) / 1e12) <= 1e-6 * d["value"]
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour on a box with no GPU")
def test_repo_arm_fails_loudly_without_a_gpu():
    r = _run("--steps", "1", "--warmup", "1", "--no-cpu-baseline", "--no-parity", "--no-sustained", timeout=300)
    assert r.returncode != 0
    assert not [ln for ln in r.stdout.splitlines() if ln.startswith("{")]      # no benchmark line from a fallback
