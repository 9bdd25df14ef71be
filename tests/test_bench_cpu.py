"""CPU test of the benchmark's reference arm: `bench.py --impl reference` times the reference CPU backend (the oracle library)
on a bounded sample and prints one JSON line with the keys the benchmark contract names.  No GPU involved."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line(built_library):
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                          "--ref-rows", "8"], capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    out = json.loads(lines[0])
    assert out["impl"] == "reference" and out["metric"] == "linear_layer_tflops" and out["unit"] == "TFLOP/s"
    assert out["higher_is_better"] is True and out["n_gpus"] == 1 and out["steps"] == 1
    assert out["value"] > 0 and out["ms_per_step"] > 0
    base = out["cpu_baseline"]
    assert base["kind"] in ("reference", "port") and base["cores"] >= 1 and base["value"] == out["value"]
    e2e = out["e2e"]
    assert e2e["value"] == out["value"] and e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0
    assert "workload" in out["config"]
