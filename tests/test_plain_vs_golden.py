"""The plain implementation against the reference's own model code (no GPU).

tests/golden/tiny_<name>.npz hold logits that the reference's Qwen2 class produced on the CPU
(scalar attention and kernels, float32) for the tiny random models A and B: after a whole prompt,
after single decode steps, for every row of a batch, and for a mixed batch of two sequences
(tests/golden/make_golden.py made them).  The plain float64 implementation must agree with them to
float32 rounding.  The weights are regenerated from the seed by the engine's own counter-based generator,
whose arithmetic is fixed (csrc/random_weights.h); a hash that no longer matches the golden file's is a
failure: either the generator or the golden files must be put right (tests/golden/make_golden.py).
"""
import hashlib
import os

import numpy as np
import pytest
import torch

from conftest import ROOT, TINY
from plain import qwen2_plain as plain


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_the_reference_model(model_dirs, name):
    golden = np.load(os.path.join(ROOT, "tests", "golden", f"tiny_{name}.npz"))
    config, weights = plain.read_model(model_dirs[name])
    digest = hashlib.sha256()
    for key in sorted(weights):
        digest.update(key.encode())
        digest.update(weights[key].float().numpy().astype("<f4").tobytes())
    assert digest.hexdigest() == str(golden["weights_sha256"]), \
        "the seeded weights differ from those the golden files were made with"
    sequences = {0: [int(t) for t in golden["first"]], 1: [int(t) for t in golden["second"]]}
    full = {s: plain.logits_of(config, weights, tokens).float().numpy() for s, tokens in sequences.items()}
    expected = np.stack([full[int(s)][int(p)] for s, p in zip(golden["row_sequence"], golden["row_position"])])
    got = golden["logits"]
    scale = float(np.abs(got).max())
    worst = float(np.abs(expected - got).max())
    assert worst < 2e-6 * max(scale, 1.0), (worst, scale)
    assert (expected.argmax(-1) == got.argmax(-1)).all()


def test_plain_sampler_draws_what_the_reference_sampler_draws():
    """tests/golden/sampler.npz: picks of the reference's sample_token for greedy rows (one with a tie, one
    after a penalty), temperature draws from several seeds, each cut alone and together, and the penalty over a
    window and over the whole history.  The plain sampler walks the same generator and must pick the same
    tokens; where the reference exponentiates with its AVX2 kernel a draw within 1e-6 of a boundary may fall
    the other way, so a stray pick in a hundred is let through for the drawn rows, none for the greedy ones."""
    golden = np.load(os.path.join(ROOT, "tests", "golden", "sampler.npz"))
    logits = golden["logits"]
    drawn = agreed = 0
    for line, picks in zip(golden["cases"], golden["picks"]):
        fields = str(line).split()
        row, draws, seed = int(fields[0]), int(fields[1]), int(fields[2])
        temperature, top_k, top_p, min_p, penalty = float(fields[3]), int(fields[4]), float(fields[5]), float(fields[6]), float(fields[7])
        window, history = int(fields[8]), [int(t) for t in fields[10:10 + int(fields[9])]]
        rng = plain.PlainXorShift32(seed)
        scores = plain.penalize_plain(logits[row], history, penalty, window)
        for d in range(draws):
            if temperature <= 0.0 or (top_k <= 0 and top_p >= 1.0 and min_p <= 0.0):
                token = plain.sample_plain(scores, temperature, rng)
            else:
                token = plain.sample_cuts_plain(scores, temperature, top_k, top_p, min_p, float(rng.next()))
            if temperature <= 0.0:
                assert token == int(picks[d]), str(line)
            else:
                drawn += 1
                agreed += token == int(picks[d])
    assert drawn > 300 and agreed >= drawn - drawn // 100, (agreed, drawn)
