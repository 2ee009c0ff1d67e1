"""The random-weights generator: the host loop of the package against the tests' own numpy restatement,
bit for bit, and what the values look like."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import TINY
from plain import random_plain


@pytest.mark.parametrize("seed,name,shape", [(0, "model.layers.3.mlp.up_proj.weight", (333, 1001)), (5, "x", (7,)),
                                             (123456789, "lm_head.weight", (5, 3, 11)), (2**40 + 3, "ü", (70001,))])
def test_host_fill_equals_the_numpy_restatement(seed, name, shape):
    from aegean_tge_b200.weights import normal, random_tensor, uniform
    for draw, plain_draw in ((normal(0.02), ("normal", 0.02)), (normal(1.5), ("normal", 1.5)),
                             (uniform(0.9, 1.1), ("uniform", 0.9, 1.1)), (uniform(-2.0, 0.5), ("uniform", -2.0, 0.5))):
        want = random_plain.tensor(seed, name, shape, plain_draw)
        got = random_tensor(name, shape, draw, seed, torch.float32, "cpu").numpy()
        assert got.dtype == np.float32 and np.array_equal(got.view(np.uint32), want.view(np.uint32))
        rounded = random_tensor(name, shape, draw, seed, torch.bfloat16, "cpu").float().numpy()
        assert np.array_equal(rounded.view(np.uint32), random_plain.to_bfloat16(want).view(np.uint32))


def test_a_run_of_a_tensor_is_that_run():
    whole = random_plain.tensor(3, "y", (1000, 77), ("normal", 0.5)).ravel()
    assert np.array_equal(random_plain.tensor(3, "y", (1000, 77), ("normal", 0.5), first=12345, count=40001),
                          whole[12345:12345 + 40001])


def test_distributions():
    x = random_plain.tensor(1, "w", (1 << 20,), ("normal", 0.02)).astype(np.float64)
    assert abs(x.mean()) < 1e-4 and abs(x.std() - 0.02) < 1e-4
    assert 2.7 < ((x - x.mean()) ** 4).mean() / x.var() ** 2 < 3.0      # a sum of eight uniforms: 2.85
    u = random_plain.tensor(1, "n", (1 << 20,), ("uniform", 0.9, 1.1)).astype(np.float64)
    assert u.min() >= np.float32(0.9) - 1e-7 and u.max() <= np.float32(1.1) and abs(u.mean() - 1.0) < 1e-3 and abs(u.std() - 0.2 / 12 ** 0.5) < 1e-3
    # other names and seeds give other tensors
    assert not np.array_equal(random_plain.tensor(1, "w", (64,), ("normal", 0.02)), random_plain.tensor(2, "w", (64,), ("normal", 0.02)))
    assert not np.array_equal(random_plain.tensor(1, "w", (64,), ("normal", 0.02)), random_plain.tensor(1, "v", (64,), ("normal", 0.02)))


@pytest.mark.parametrize("name", ["A", "B"])
def test_a_written_model_folder_holds_the_restated_model(model_dirs, name):
    """``write_random_model`` (what ``tge make-random`` calls) against the numpy plan of the same architecture."""
    from safetensors import safe_open
    config, seed = TINY[name]
    want = random_plain.qwen2_weights(config, seed)
    with safe_open(os.path.join(model_dirs[name], "model.safetensors"), framework="np") as handle:
        assert sorted(handle.keys()) == sorted(want)
        for key in handle.keys():
            assert np.array_equal(handle.get_tensor(key), want[key]), key
    with open(os.path.join(model_dirs[name], "config.json")) as handle:
        assert json.load(handle)["vocab_size"] == config["vocab_size"]


@pytest.mark.gpu
@pytest.mark.parametrize("count,first", [(1, 0), (7, 3), (4097, 0), (333 * 1001, 0), (100003, 999)])
def test_device_fill_equals_the_numpy_restatement(count, first):
    """The fill kernel at odd sizes and, through a view that starts at an odd element, odd addresses."""
    from aegean_tge_b200 import ops
    from aegean_tge_b200.weights import normal, tensor_key, uniform
    lib = ops.core()
    for draw, plain_draw in ((normal(0.02), ("normal", 0.02)), (uniform(0.9, 1.1), ("uniform", 0.9, 1.1)),
                             (uniform(-2.0, 0.5), ("uniform", -2.0, 0.5))):
        want = random_plain.tensor(9, "some.tensor", (first + count,), plain_draw, first=first, count=count)
        for dtype in (torch.float32, torch.bfloat16):
            for shift in (0, 1):
                buffer = torch.zeros(count + shift + 1, dtype=dtype, device="cuda")
                out = buffer[shift:shift + count]
                ops._check(lib.tge_random_fill(out.data_ptr(), int(dtype == torch.bfloat16), count, first,
                                               tensor_key(9, "some.tensor"), draw.kind, draw.scale, draw.base,
                                               draw.span, ops._stream()), lib)
                got = out.float().cpu().numpy()
                expect = want if dtype == torch.float32 else random_plain.to_bfloat16(want)
                assert np.array_equal(got.view(np.uint32), expect.view(np.uint32)), (dtype, shift, plain_draw)
                assert float(buffer[shift + count]) == 0.0 and (shift == 0 or float(buffer[0]) == 0.0)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["B", "E"])
def test_a_model_drawn_on_the_device_is_the_model_written_to_disk(model_dirs, name):
    """``Engine(random_config=, seed=)`` and ``Engine(model_dir)`` of ``write_random_model`` with the same seed:
    the same weights, so the same logits bit for bit in float32."""
    from aegean_tge_b200 import Engine
    from aegean_tge_b200.engine.batch import Portion
    config, seed = TINY[name]
    tokens = [(7 * i + 3) % config["vocab_size"] for i in range(40)]
    rows = []
    for kwargs in ({"model_dir": model_dirs[name]}, {"random_config": config, "seed": seed}):
        engine = Engine(dtype="float32", context=128, max_tokens=256, max_requests=2, **kwargs)
        rows.append(engine.runner.step([Portion("r", tokens, list(range(len(tokens))))]).cpu())
        del engine
    assert torch.equal(rows[0], rows[1])
