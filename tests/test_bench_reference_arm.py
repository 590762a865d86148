"""The benchmark's reference arm runs without a GPU: it times the reference's own CPU attention (or the oracle
port where the reference library was not built) on the host cores and prints one JSON line with the keys the
benchmark contract names."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    lines = [l for l in out.stdout.strip().splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "fwd_attention_tflops" and line["unit"] == "TFLOP/s"
    assert line["value"] > 0 and line["higher_is_better"] is True and line["gpu_launches"] == 0
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "config 2" in line["config"]["workload"]


def test_traffic_file_names_its_captures():
    t = json.load(open(os.path.join(ROOT, "profiles", "ncu_traffic.json")))
    for name, e in t.items():
        assert e["bytes_per_launch"] > 0
        src = e["source"].split(":")[0]
        assert os.path.exists(os.path.join(ROOT, src)), src
