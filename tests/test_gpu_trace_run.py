"""bin/trace_run as a user runs it: a child process fed steps on standard input, answering
"done <step>" after each, writing <step>.f32 files; checked against the plain implementation."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.helpers import CONFIGS, check_against_plain, model_folder, requests_for

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("tag,dtype", [("tiny_a", "float32"), ("tiny_b", "bfloat16")])
def test_trace_run_replays_a_batch(tag, dtype, tmp_path):
    vocab = CONFIGS[tag]["vocab_size"]
    a, b, c = requests_for(tag, [40, 70, 9], seed=31)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}, {"id": "b", "tokens": b[:64], "want": []},
                                {"id": "c", "tokens": c, "want": [8]}], "end": ["c"]},
    ]
    for i in range(6):
        steps.append({"step": i + 1, "entries": [{"id": "a", "tokens": [a[30 + i]], "want": [0]},
                                                 {"id": "b", "tokens": [b[64 + i]], "want": [0]}],
                      "end": ["a"] if i == 5 else []})
    steps.append({"step": 7, "entries": [{"id": "b", "tokens": [], "want": []}][:0], "end": ["b"]})
    steps.append({"step": 8, "entries": [{"id": 5, "tokens": c, "want": list(range(9))}], "end": [5]})  # a slot used again
    proc = subprocess.Popen(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_folder(tag)), "--dtype", dtype, "--out",
         str(tmp_path), "--max-tokens", "256"],
        stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, cwd=tmp_path)
    for step in steps:
        proc.stdin.write(json.dumps(step) + "\n")
        proc.stdin.flush()
        assert proc.stdout.readline().strip() == f"done {step['step']}"  # the next step only after this line
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0

    def read(step, n):
        data = np.fromfile(tmp_path / f"{step}.f32", dtype="<f4")
        assert data.size == n * vocab
        return torch.from_numpy(data.reshape(n, vocab))

    first = read(0, 3)
    check_against_plain(tag, dtype, a, [0, 29], first[:2], "trace step 0, request a")
    check_against_plain(tag, dtype, c, [8], first[2:], "trace step 0, request c")
    for i in range(6):
        rows = read(i + 1, 2)
        check_against_plain(tag, dtype, a, [30 + i], rows[:1], f"trace step {i + 1}, request a")
        check_against_plain(tag, dtype, b, [64 + i], rows[1:], f"trace step {i + 1}, request b")
    assert not (tmp_path / "7.f32").exists()  # nothing was wanted in that step
    check_against_plain(tag, dtype, c, list(range(9)), read(8, 9), "trace step 8, slot used again")
