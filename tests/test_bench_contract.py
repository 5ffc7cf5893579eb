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
    assert line["cpu_baseline"]["kind"] in ("reference", "port")
    assert line["cpu_baseline"]["value"] == line["value"]
    assert line["cpu_baseline"]["cores"] >= 1 and "sample" in line["cpu_baseline"]
    assert line["e2e"] == {"value": line["value"], "unit": "ms", "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
    assert "workload" in line["config"] and "model" not in line["config"]


def test_bench_refuses_an_unknown_workload():
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--workload", "nope"],
                          capture_output=True, text=True, timeout=120, cwd=str(ROOT))
    assert proc.returncode != 0


def test_reference_arm_never_loads_the_cuda_library():
    """The reference arm's workload module runs without importing this repository's package,
    so the timed process maps no libdexter_b200.so; it uses every host core even when the
    launcher exported OMP_NUM_THREADS=1 (as torch.distributed.run does)."""
    code = ("import os, sys; sys.path.insert(0, %r); os.environ['OMP_NUM_THREADS'] = '1';"
            "import bench; from oracle import ref_workload as r;"
            "kind, linears, run = r.build_block('5b'); n = r.use_all_host_threads();"
            "maps = open('/proc/self/maps').read();"
            "assert 'dexter_labs_b200' not in sys.modules and 'libdexter_b200' not in maps;"
            "assert n == len(os.sched_getaffinity(0)), n; print(kind, len(linears))" % str(ROOT))
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split()[1] == "10"


def test_both_arms_print_the_same_config():
    import bench

    for n in (1, 2, 8):
        assert bench.workload_config(n, "fused") == bench.workload_config(n, "fused")
    assert bench.workload_config(8)["collectives"] != "none" and bench.workload_config(1)["collectives"] == "none"
