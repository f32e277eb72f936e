"""bench.py prints ONE JSON line with the agreed keys: the reference arm (CPU oracle) here, the GPU
arm on a B200."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE_KEYS = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
             "vs_baseline", "dtype", "data", "config", "e2e"}


def _run(args, timeout):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py")] + args, capture_output=True, text=True,
                         timeout=timeout, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, lines
    return json.loads(lines[0])


def test_reference_arm_line():
    d = _run(["--impl", "reference", "--steps", "1", "--warmup", "0"], timeout=280)
    assert BASE_KEYS <= set(d), BASE_KEYS - set(d)
    assert d["impl"] == "reference" and d["metric"] == "encoder_tokens_per_s" and d["unit"] == "tokens/s"
    assert d["higher_is_better"] is True and d["vs_baseline"] is None and d["value"] > 0
    assert "workload" in d["config"]
    cb = d["cpu_baseline"]
    # the reference's own module when the build placed it under oracle/_ref, else the restatement
    from oracle import ref_runner
    assert cb["kind"] == ("reference" if ref_runner.available() else "port")
    assert cb["cores"] >= 1 and "whole seed-0 batch" in cb["sample"] and cb["value"] == d["value"]
    assert d["config"]["tokens"] == 16512 and d["config"]["sequences"] == 8
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


@pytest.mark.gpu
def test_gpu_arm_line():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    d = _run(["--steps", "2", "--warmup", "3"], timeout=280)
    assert BASE_KEYS | {"roofline", "cpu_baseline", "gpu_launches", "clocks"} <= set(d)
    assert d["n_gpus"] == 1 and d["steps"] == 2 and d["warmup"] == 4 and d["value"] > 1e5  # 4 rotating batches
    assert d["gpu_launches"] >= 2 * 70  # 6 kernels per layer + embeddings + position ids per step
    assert d["dtype"] == "f16" and d["data"] == "synthetic"
    r = d["roofline"]
    assert r["bound"] == "tensor" and r["unit"] == "TFLOP/s" and 0 < r["frac"] < 1.2
    assert abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9
    e = d["e2e"]
    assert e["value"] > 1e5 and e["h2d_bytes_per_step"] > 0 and e["d2h_bytes_per_step"] > 8 * 1024 * 768 * 2
    assert e["value"] != d["value"]
    assert d["config"]["tokens"] == 16512 and d["host_work_ms_per_step"] > 0
    assert d["cpu_baseline"]["kind"] in ("port", "reference") and d["cpu_baseline"]["value"] > 0
    assert "whole seed-0 batch" in d["cpu_baseline"]["sample"]
    assert set(d["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}
