"""The parts of bench.py's contract that need no GPU: more than one GPU is refused with one line and
exit code 2; the reference arm prints one record, drives the reference's own engine and names the own arm's config."""

import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=120)


def test_more_than_one_gpu_is_refused():
    out = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert out.returncode == 2
    lines = [line for line in out.stdout.splitlines() if line.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_prints_one_record():
    """Without a GPU the arm says so (or that no copy of the reference is there) in one line and exits 0."""
    out = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert out.returncode == 0
    record = json.loads(out.stdout.strip().splitlines()[-1])
    assert record["impl"] == "reference"
    if "unavailable" in record:
        assert "\n" not in record["unavailable"] and ("CUDA" in record["unavailable"] or "copy" in record["unavailable"])
    else:
        assert record["config"]["hidden_size"] == 1024 and record["value"] > 0


def test_reference_arm_drives_the_reference_engine_and_names_the_same_config():
    """The arm's harness, run here on the CPU on a shrunken model: it times the reference's own
    Engine.generate and prints the keys and the config record of the own arm."""
    import argparse

    sys.path.insert(0, str(ROOT))
    import bench

    if bench.reference_folder() is None:
        pytest.skip("no copy of the reference beside the repository")
    args = argparse.Namespace(batch=2, steps=3, warmup=3, layers=2)
    small = {"hidden_size": 32, "intermediate_size": 64, "num_attention_heads": 2, "num_key_value_heads": 1,
             "head_dim": 16, "vocab_size": 97}
    record = bench.run_reference(args, device="cpu", sizes=small, prompt_len=12, prefill_tokens=16, batches=(1,))
    assert "unavailable" not in record, record
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "dtype",
                "config", "e2e", "prefill", "roofline", "points", "clocks"):
        assert key in record, key
    assert record["impl"] == "reference" and record["steps"] == 3 and record["value"] > 0
    assert record["config"] == bench.config_record(2, 2, bench.peaks()[1])
    assert len(record["config"]) <= 20 and all(not isinstance(v, (dict, list)) for v in record["config"].values())


def test_reference_arm_imports_nothing_of_the_package():
    import ast

    tree = ast.parse((ROOT / "bench.py").read_text())
    arm = [node for node in ast.walk(tree) if isinstance(node, (ast.ClassDef, ast.FunctionDef))
           and node.name in ("ReferenceArm", "run_reference", "reference_folder")]
    assert len(arm) == 3
    for node in arm:
        for inner in ast.walk(node):
            if isinstance(inner, ast.ImportFrom):
                assert not (inner.module or "").startswith("gtar_kimik3_public_b200"), inner.module
            if isinstance(inner, ast.Import):
                assert all(not a.name.startswith("gtar_kimik3_public_b200") for a in inner.names)
