"""bin/trace_run as a user runs it: a subprocess fed steps on standard input."""
import json
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, TINY
from helpers import model_tol, rel_error
from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu


def _replay(model_dir, dtype, steps, out_dir, max_tokens):
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype",
                             dtype, "--out", out_dir, "--max-tokens", str(max_tokens)],
                            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for step in steps:
        proc.stdin.write(json.dumps(step) + "\n")
        proc.stdin.flush()
        answer = proc.stdout.readline().strip()
        assert answer == f"done {step['step']}", answer
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_trace_run_mixed_trace(model_dirs, tmp_path, name, dtype):
    config, seed = TINY[name]
    rnd = random.Random(seed + 5)
    tokens = {r: [rnd.randrange(config["vocab_size"]) for _ in range(n)] for r, n in (("a", 75), ("b", 40), ("c", 66))}
    raw, weights = plain.read_model(model_dirs[name])
    ref = {r: plain.logits_of(raw, weights, t).float() for r, t in tokens.items()}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": tokens["a"][:40], "want": [39]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": tokens["a"][40:42], "want": [0, 1]},
                                {"id": "b", "tokens": tokens["b"][:38], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": tokens["b"][38:39], "want": [0]}], "end": []},
        {"step": 3, "entries": [{"id": "b", "tokens": tokens["b"][39:40], "want": [0]},
                                {"id": "a", "tokens": tokens["a"][42:75], "want": [32, 0]}], "end": ["a", "b"]},
        {"step": 4, "entries": [{"id": "c", "tokens": tokens["c"], "want": list(range(66))}], "end": ["c"]},
    ]
    out_dir = str(tmp_path / "out")
    _replay(model_dirs[name], dtype, steps, out_dir, max_tokens=192)     # a (128) + b (64): c reuses their pages
    vocab = config["vocab_size"]
    load = lambda s: torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{s}.f32"), dtype="<f4").reshape(-1, vocab))
    tol = model_tol(dtype, name)
    assert rel_error(load(0), ref["a"][[39]]) < tol
    assert rel_error(load(1), ref["a"][[40, 41]]) < tol
    assert rel_error(load(2), ref["b"][[38]]) < tol
    assert rel_error(load(3), torch.cat([ref["b"][[39]], ref["a"][[74, 42]]])) < tol
    assert rel_error(load(4), ref["c"]) < tol
    assert not os.path.exists(os.path.join(out_dir, "5.f32"))
