"""The benchmark's output contract: one JSON line with the agreed keys. The reference arm runs on the host and is
checked here without a GPU; the product arm is checked on a B200."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE_KEYS = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
             "vs_baseline", "dtype", "data", "config", "e2e"}


def run_bench(*args):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                         timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, out.stdout
    return json.loads(lines[0])


def test_reference_arm_prints_one_contract_line(built):
    d = run_bench("--impl", "reference", "--steps", "2", "--warmup", "1", "--flat", str(64 << 20))
    assert BASE_KEYS <= set(d) and d["impl"] == "reference"
    assert d["metric"] == "fused_allreduce_adamw_algorithmic_GBps" and d["unit"] == "GB/s" and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] == 1
    assert d["e2e"] == {"value": d["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"] and "model" not in d["config"]


def test_reference_arm_under_torchrun_only_rank_zero_reports(built):
    """Launched the way the scaling runs launch it (one process per rank): rank 0 times the host path with one
    thread per rank, the other ranks leave quietly."""
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "bench.py"),
                          "--impl", "reference", "--gpus", "2", "--steps", "2", "--warmup", "1", "--flat", str(64 << 20)],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    assert lines[0]["n_gpus"] == 2 and lines[0]["cpu_baseline"]["cores"] == 2 and lines[0]["impl"] == "reference"


@pytest.mark.gpu
def test_product_arm_prints_one_contract_line(cuda):
    d = run_bench("--flat", str(64 << 20), "--steps", "5", "--warmup", "3", "--e2e-steps", "1")
    assert BASE_KEYS | {"roofline", "cpu_baseline", "gpu_launches", "clocks"} <= set(d)
    assert d["n_gpus"] == 1 and d["gpu_launches"] == 5 and d["vs_baseline"] is None and d["dtype"] == "f32"
    r = d["roofline"]
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and 0.3 < r["frac"] < 1.1 and r["traffic"] > 0
    assert abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9
    e = d["e2e"]
    assert e["h2d_bytes_per_step"] == 64 << 20 and e["d2h_bytes_per_step"] == 64 << 20 and 0 < e["value"] < d["value"]
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["value"] > 0
    assert set(d["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}
