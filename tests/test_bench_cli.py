"""The benchmark's command-line contract: one JSON line with the agreed keys."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
COMMON = ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
          "vs_baseline", "dtype", "data", "config", "e2e", "cpu_baseline")


def _run(*args):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                         timeout=900, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, out.stdout[-2000:]
    return json.loads(lines[0])


def test_reference_arm_prints_one_json_line():
    d = _run("--impl", "reference", "--workload", "flat20", "--vsw", "2", "--steps", "2", "--warmup", "1")
    for key in COMMON:
        assert key in d, key
    assert d["impl"] == "reference" and d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["value"] == d["value"] > 0
    assert d["config"]["workload"] == "flat20" and d["unit"] == "samples/s"


@pytest.mark.gpu
def test_default_arm_prints_one_json_line():
    d = _run("--workload", "flat22", "--steps", "20", "--warmup", "3", "--cpu-steps", "2")
    for key in COMMON + ("roofline", "gpu_launches", "clocks", "kernels"):
        assert key in d, key
    r = d["roofline"]
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and 0 < r["frac"] < 1.5 and r["achieved"] > 0
    assert abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9
    assert d["gpu_launches"] >= 20 and d["value"] > 0 and d["e2e"]["value"] > 0
    assert d["e2e"]["h2d_bytes_per_step"] == 4 * 4 * (1 << 22) and d["e2e"]["d2h_bytes_per_step"] == 4
    assert d["cpu_baseline"]["value"] > 0 and d["dtype"] == "f32" and -1.0 <= d["cosine"] <= 1.0


def test_reference_arm_under_torchrun_with_two_ranks():
    """Launched the way a multi-GPU run is: rank 0 alone runs the CPU ranks (which must ignore
    the launcher's rendezvous environment) and prints the line; the other rank exits 0."""
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29571", os.path.join(ROOT, "bench.py"),
                          "--impl", "reference", "--gpus", "2", "--workload", "flat20", "--vsw", "2",
                          "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 2 and d["value"] > 0
    assert "2 gloo rank(s)" in d["cpu_baseline"]["sample"]
