"""GPU: one short run of bench.py; the JSON line carries every key of the benchmark contract."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_bench_line_has_the_contract_keys():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "6", "--warmup", "3",
                          "--e2e-steps", "2", "--no-small", "--no-ref-cuda"],
                         capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "roofline", "cpu_baseline", "e2e", "gpu_launches", "clocks"):
        assert key in line, key
    assert line["steps"] == 6 and line["warmup"] == 3 and line["n_gpus"] == 1
    assert line["dtype"] == "f32" and line["data"] == "synthetic" and line["scaling"] == "weak"
    assert line["config"]["workload"].startswith("cfg2: 131072x256")
    assert line["device_status"] == "ok"
    roof = line["roofline"]
    assert roof["bound"] == "hbm" and roof["unit"] == "GB/s" and roof["peak"] > 0
    assert abs(roof["frac"] - roof["achieved"] / roof["peak"]) < 1e-9
    assert 0.5 < roof["frac"] < 1.2            # the kernel did the work, and at memory speed
    assert roof["traffic"] is None or roof["traffic"] > 0.9 * roof["algorithmic_bytes"]
    cpu = line["cpu_baseline"]
    assert cpu["kind"] in ("reference", "port") and cpu["cores"] >= 1 and cpu["value"] > 0 and cpu["sample"]
    e2e = line["e2e"]
    assert e2e["value"] > 0 and e2e["unit"] == line["unit"]
    assert e2e["h2d_bytes_per_step"] == 16 * 131072 * 256 and e2e["d2h_bytes_per_step"] > 0
    assert e2e["value"] < line["value"]        # host copies inside the timed region
    assert line["gpu_launches"] >= line["steps"]
    assert set(("sm_mhz", "sm_max_mhz", "reasons")) <= set(line["clocks"])
