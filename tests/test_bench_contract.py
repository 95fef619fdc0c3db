"""The one-line JSON contract of bench.py: the CPU (reference) arm runs anywhere; the GPU arm needs a B200."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, timeout=600):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py")] + args, capture_output=True, text=True,
                         timeout=timeout, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, out.stdout[-2000:]
    return json.loads(lines[0])


def test_reference_arm_line():
    """`--impl reference`: the CPU implementation of the path on the host cores, same metric and unit, no GPU."""
    d = _run(["--impl", "reference", "--config", "1", "--steps", "2", "--warmup", "1"])
    assert d["impl"] == "reference" and d["metric"] == "sru_fwd_bwd_tokens_per_sec" and d["unit"] == "tokens/s"
    assert d["higher_is_better"] is True and d["value"] > 0 and d["steps"] == 2
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("port", "reference") and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"] and "model" not in d["config"]


@pytest.mark.gpu
def test_gpu_arm_line():
    """The GPU arm's line carries every key of the contract, with a roofline object for the dominant kernel class,
    an end-to-end figure that counts its host copies, the launches of this library and the clock record."""
    d = _run(["--config", "2", "--steps", "3", "--warmup", "3", "--cpu-sample-batch", "2"])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "clocks", "roofline", "cpu_baseline",
                "kernels", "check"):
        assert key in d, key
    assert d["n_gpus"] == 1 and d["steps"] == 3 and d["warmup"] == 3 and d["value"] > 0 and d["vs_baseline"] is None
    assert abs(d["value"] - 256 * 64 / (d["ms_per_step"] / 1e3)) <= 1e-6 * d["value"]
    e = d["e2e"]
    assert e["value"] > 0 and e["h2d_bytes_per_step"] >= 256 * 64 * 512 * 4 and e["d2h_bytes_per_step"] >= 4
    r = d["roofline"]
    assert r["bound"] in ("hbm", "tensor") and r["unit"] in ("GB/s", "TFLOP/s") and r["peak"] > 0
    assert abs(r["frac"] - r["achieved"] / r["peak"]) <= 1e-9 and (r["traffic"] is None or r["traffic"] > 0)
    assert d["gpu_launches"] > 0 and d["gpu_launches"] % 3 == 0
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("port", "reference") and cb["value"] > 0 and cb["cores"] >= 1
    assert "workload" in d["config"] and d["dtype"] == "bf16" and d["data"] == "synthetic"
    assert d["clocks"] is None or "sm_mhz" in d["clocks"]
