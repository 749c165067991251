"""The one JSON line bench.py prints: keys and meanings the driver of the benchmark relies on.  The reference arm
(CPU only) runs anywhere; the CUDA arm needs a GPU."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, out.stdout[-2000:]
    return json.loads(lines[0])


def _common(d, steps):
    assert d["metric"] == "cost_volume_fwd_bwd_voxel_views_per_s" and d["unit"] == "voxel*views/s"
    assert d["higher_is_better"] is True and d["vs_baseline"] is None and d["data"] == "synthetic"
    assert d["n_gpus"] == 1 and d["steps"] == steps and d["value"] > 0 and d["ms_per_step"] > 0
    assert d["config"]["workload"].startswith("c1_mvsnet: CostVolume fwd+bwd fp32, B=1 per GPU, V=3, C=32, 128x160, D=192")
    assert d["dtype"] == "f32"


def test_reference_arm_line():
    import bench
    d = _run("--impl", "reference", "--steps", "1", "--warmup", "0")
    _common(d, 1)
    assert d["impl"] == "reference" and d["gpu_launches"] == 0
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["sample"] and cb["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    # both arms describe the workload with the same dictionary
    assert d["config"] == bench.cost_volume_config("c1_mvsnet", "batch", 1, 2, 32, 128, 160, 192)


@pytest.mark.gpu
def test_cuda_arm_line():
    import bench
    d = _run("--steps", "5", "--warmup", "3")
    _common(d, 5)
    assert "impl" not in d or d["impl"] != "reference"
    assert d["warmup"] >= 3 and d["scaling"] == "weak" and d["gpu_launches"] == 3 * 5
    assert d["config"] == bench.cost_volume_config("c1_mvsnet", "batch", 1, 2, 32, 128, 160, 192)
    r = d["roofline"]
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and r["peak"] > 0 and r["achieved"] > 0
    assert abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9
    assert r["traffic"] is None or r["traffic"] > 1e8        # recorded DRAM bytes, or null when the kernels are newer
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["value"] > 0 and cb["sample"]
    e = d["e2e"]
    assert e["unit"] == d["unit"] and 0 < e["value"] < d["value"]           # host copies inside the timed region
    assert e["h2d_bytes_per_step"] > 5e8 and e["d2h_bytes_per_step"] > 5e8   # cost_grad in, cost out
    c = d["clocks"]
    assert c["sm_mhz"] > 0 and c["sm_max_mhz"] >= c["sm_mhz"] and isinstance(c["reasons"], list)
