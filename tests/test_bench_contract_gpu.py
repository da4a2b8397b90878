"""bench.py prints exactly one JSON line on stdout with the keys its readers rely on."""
import json
import os
import subprocess
import sys

import pytest

from tests._util import ROOT

pytestmark = pytest.mark.gpu


def _run(*args):
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                         timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, lines
    return json.loads(lines[0])


def test_b200_arm_line():
    d = _run("--workload", "cfg2_small", "--steps", "3", "--warmup", "3", "--no-cpu-baseline")
    for k in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
              "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "clocks", "roofline"):
        assert k in d, k
    assert d["n_gpus"] == 1 and d["steps"] == 3 and d["warmup"] == 3 and d["higher_is_better"] is True
    assert d["scaling"] == "strong" and d["config"]["global_batch"] == 4
    assert d["value"] > 0 and d["ms_per_step"] > 0 and d["gpu_launches"] > 0 and d["dtype"] == "f32"
    assert "workload" in d["config"]
    e = d["e2e"]
    assert e["value"] > 0 and e["h2d_bytes_per_step"] > 0 and e["d2h_bytes_per_step"] > 0
    assert e["value"] != d["value"]
    r = d["roofline"]
    for k in ("bound", "achieved", "peak", "unit", "frac", "traffic"):
        assert k in r, k
    assert abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9


def test_reference_arm_line():
    d = _run("--impl", "reference", "--workload", "cfg2_small", "--steps", "1", "--warmup", "0")
    assert d["impl"] == "reference" and d["value"] > 0
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1
    assert d["cpu_baseline"]["cpu_sample_N"] >= 32 and d["scaling"] == "strong"
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
