"""The parts of bench.py's contract that need no GPU: more than one GPU is refused with one line and
exit code 2; the reference arm reports that the reference cannot be installed and exits 0."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=120)


def test_more_than_one_gpu_is_refused():
    out = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert out.returncode == 2
    lines = [line for line in out.stdout.splitlines() if line.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_is_unavailable():
    out = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert out.returncode == 0
    record = json.loads(out.stdout.strip().splitlines()[-1])
    assert record["impl"] == "reference" and "unavailable" in record and "\n" not in record["unavailable"]
