"""bench.py without a GPU: the reference arm (the CPU port timed on the host cores) prints one JSON
line with the contract's keys, and the GPU arm's command line is the documented one."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def run_bench(*args):
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    return res.stdout


def test_reference_arm_prints_the_contract_line():
    out = run_bench("--impl", "reference", "--steps", "1", "--warmup", "1", "--cpu-seconds", "1")
    lines = [ln for ln in out.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "GB/s" and d["higher_is_better"] is True
    assert d["n_gpus"] == 1 and d["steps"] == 1 and d["value"] > 0 and d["vs_baseline"] is None
    assert d["config"]["workload"].startswith("c2")
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_command_line_has_the_contract_flags():
    out = run_bench("--help")
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--workload", "--no-torch", "--no-triton-ref"):
        assert flag in out
