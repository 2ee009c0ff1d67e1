"""The plain implementation checked against itself (no GPU)."""
import random

import numpy as np
import torch

from conftest import TINY
from plain import qwen2_plain as plain


def test_prefix_logits_do_not_change_when_tokens_are_appended(model_dirs):
    """Causality: the logits of a prefix equal the first rows of the longer sequence's logits."""
    config, weights = plain.read_model(model_dirs["B"])
    rnd = random.Random(0)
    tokens = [rnd.randrange(config["vocab_size"]) for _ in range(24)]
    full = plain.logits_of(config, weights, tokens)
    part = plain.logits_of(config, weights, tokens[:9])
    assert float((full[:9] - part).abs().max()) < 1e-12


def test_rope_tables_are_float32_angles():
    cos, sin = plain.rope_tables(1000000.0, 32, 50)
    assert cos.shape == (50, 16) and float(cos[0].min()) == 1.0 and float(sin[0].abs().max()) == 0.0
    freq1 = np.float32(np.float64(np.float32(1e6)) ** np.float64(np.float32(-2.0) / np.float32(32)))
    assert abs(float(cos[7, 1]) - np.cos(np.float64(np.float32(7) * freq1))) < 1e-15
    # the package's tables are the same numbers (built by other code)
    from aegean_tge_b200.parts.rope import rotary_tables
    c2, s2 = rotary_tables(1000000.0, 32, 50)
    assert torch.equal(c2, cos.float()) and torch.equal(s2, sin.float())


def test_attention_is_a_convex_mix_and_groups_share_kv():
    gen = torch.Generator().manual_seed(0)
    q = torch.randn(5, 4, 8, generator=gen, dtype=torch.float64)
    k = torch.randn(5, 2, 8, generator=gen, dtype=torch.float64)
    v = torch.ones(5, 2, 8, dtype=torch.float64) * torch.tensor([1.0, 2.0])[None, :, None]
    out = plain.attention(q, k, v)
    assert torch.allclose(out[:, :2], torch.ones(5, 2, 8, dtype=torch.float64))       # heads 0,1 -> kv head 0
    assert torch.allclose(out[:, 2:], 2 * torch.ones(5, 2, 8, dtype=torch.float64))   # heads 2,3 -> kv head 1
    first = plain.attention(q[:1], k[:1], torch.randn(1, 2, 8, generator=gen, dtype=torch.float64))
    assert first.shape == (1, 4, 8)


def test_sampler_rules():
    rng = plain.PlainXorShift32(0)
    assert rng.state == 0x9E3779B9                                  # seed 0 -> the fixed default
    u = [float(rng.next()) for _ in range(1000)]
    assert 0.0 <= min(u) and max(u) < 1.0 and abs(np.mean(u) - 0.5) < 0.05
    logits = np.array([0.0, 3.0, 3.0, -1.0], dtype=np.float32)
    assert plain.sample_plain(logits, 0.0, rng) == 1               # first maximum
    draws = [plain.sample_plain(logits, 1.0, rng) for _ in range(2000)]
    share = np.bincount(draws, minlength=4) / 2000
    p = np.exp(logits - 3.0); p /= p.sum()
    assert np.abs(share - p).max() < 0.05
    from aegean_tge_b200.sampling import XorShift32
    a, b = XorShift32(42), plain.PlainXorShift32(42)
    assert [a.next_uniform() for _ in range(50)] == [float(b.next()) for _ in range(50)]
