"""The reference arm of bench.py runs on the host cores alone: check the JSON line it prints."""
import json
import subprocess
import sys

from conftest import ROOT


def test_reference_arm_prints_the_contract_line():
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1",
                           "--warmup", "1"], capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference"
    assert line["metric"] == "w4a16_5b_layer_set_ms" and line["unit"] == "ms"
    assert line["higher_is_better"] is False and line["vs_baseline"] is None
    assert line["value"] > 0 and line["ms_per_step"] == line["value"]
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["value"] == line["value"]
    assert line["cpu_baseline"]["cores"] >= 1 and "sample" in line["cpu_baseline"]
    assert line["e2e"] == {"value": line["value"], "unit": "ms", "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
    assert "workload" in line["config"] and "model" not in line["config"]


def test_bench_refuses_an_unknown_workload():
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--workload", "nope"],
                          capture_output=True, text=True, timeout=120, cwd=str(ROOT))
    assert proc.returncode != 0
