"""The engine at real layer sizes against the plain implementation.

Two layers of the Qwen2.5-7B, 14B and 32B shapes (the widths, head counts, inner widths and the whole
152,064-row vocabulary of the Qwen2.5 models), random weights from the seed on both sides:
the engine draws them on the device, the oracle with the tests' own numpy restatement of the generator.
The oracle is tests/plain/qwen2_plain.py in float64.  To keep it in seconds it computes the logits of a
few runs of vocabulary rows only (the first rows, a run in the middle that starts at an odd row, and the
last rows with the ragged edge); the engine computes all of them and the same columns are compared.
For bfloat16 the oracle's matrices are the bfloat16 values the engine holds, so what is measured is the
engine's arithmetic, and the tolerance is set at about three times the error seen.
"""
import random

import numpy as np
import pytest
import torch

from helpers import rel_error
from plain import qwen2_plain as plain
from plain import random_plain

pytestmark = pytest.mark.gpu

BASE = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 2, "head_dim": 128,
        "vocab_size": 152064, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
        "max_position_embeddings": 32768, "use_sliding_window": False, "hidden_act": "silu"}
SHAPES = {
    "7B": dict(BASE, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944),
    "14B": dict(BASE, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, intermediate_size=13824),
    "32B": dict(BASE, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, intermediate_size=27648),
}
SEEDS = {"7B": 7, "14B": 14, "32B": 32}
# runs of vocabulary rows whose logits the oracle computes: (first row, rows)
HEAD_RUNS = [(0, 512), (75001, 517), (152064 - 523, 523)]
COLUMNS = torch.cat([torch.arange(a, a + n) for a, n in HEAD_RUNS])
# about three times the largest error seen (float32 9e-6, bfloat16 1.55e-2 of the largest logit)
TOL = {"float32": 3e-5, "bfloat16": 4e-2}
DTYPES = ["float32", "bfloat16"]


def _tokens(shape, count, salt):
    rnd = random.Random(1000 * SEEDS[shape] + salt)
    return [rnd.randrange(BASE["vocab_size"]) for _ in range(count)]


class _Oracle:
    """Weights of one shape from the numpy generator, and plain logits of token lists at the chosen columns."""

    def __init__(self, shape):
        self.shape, self.config, self.seed = shape, SHAPES[shape], SEEDS[shape]
        self.layers = {}
        for name, dims, role, draw in random_plain.qwen2_plan(self.config):
            if name not in ("model.embed_tokens.weight", "lm_head.weight"):
                self.layers[name] = (random_plain.tensor(self.seed, name, dims, draw), role)
        hidden = self.config["hidden_size"]
        self.head = np.concatenate([random_plain.tensor(self.seed, "lm_head.weight", (152064, hidden), ("normal", 0.02),
                                                        first=a * hidden, count=n * hidden).reshape(n, hidden)
                                    for a, n in HEAD_RUNS])
        self.cache = {}

    def _embedding_rows(self, tokens):
        hidden = self.config["hidden_size"]
        return np.stack([random_plain.tensor(self.seed, "model.embed_tokens.weight", (152064, hidden), ("normal", 0.02),
                                             first=t * hidden, count=hidden) for t in tokens])

    def logits(self, dtype, tokens):
        """float32 [len(tokens), chosen columns]"""
        global _float64_weights
        key = (dtype, tuple(tokens))
        if key not in self.cache:
            round_ = random_plain.to_bfloat16 if dtype == "bfloat16" else (lambda x: x)
            if _float64_weights[0] != (self.shape, dtype):          # one set of float64 weights in memory at a time
                _float64_weights = ((self.shape, dtype), None)
                w = {name: torch.from_numpy(round_(value) if role == "matrix" else value).double()
                     for name, (value, role) in self.layers.items()}
                w["lm_head.weight"] = torch.from_numpy(round_(self.head)).double()
                _float64_weights = ((self.shape, dtype), w)
            w = dict(_float64_weights[1])
            w["model.embed_tokens.weight"] = torch.from_numpy(round_(self._embedding_rows(tokens))).double()
            # the plain model looks rows up by token id: the tokens become 0, 1, 2, ... of this small table
            self.cache[key] = plain.logits_of(self.config, w, list(range(len(tokens)))).float()
        return self.cache[key]


_oracles = {}
_float64_weights = (None, None)


def _oracle(shape):
    if shape not in _oracles:
        _oracles[shape] = _Oracle(shape)
    return _oracles[shape]


def _engine(shape, dtype, **kw):
    from aegean_tge_b200 import Engine
    kw.setdefault("context", 1024)
    kw.setdefault("max_tokens", 2048)
    kw.setdefault("max_requests", 8)
    kw.setdefault("max_batch_tokens", 2048)
    return Engine(random_config=SHAPES[shape], seed=SEEDS[shape], dtype=dtype, **kw)


def _portion(request, tokens, want=None):
    from aegean_tge_b200.engine import Portion
    return Portion(request, tokens, list(range(len(tokens))) if want is None else want)


def _pick(logits):
    return logits[:, COLUMNS.to(logits.device)]


def _close(got, ref, dtype, what):
    error = rel_error(got, ref)
    print(f"[real shapes] {what} {dtype}: error {error:.3e} of the largest logit")
    assert error < TOL[dtype], (what, dtype, error)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", list(SHAPES))
def test_whole_then_single_tokens_then_portions(shape, dtype):
    """One request of 303 tokens: whole; 271 in one step and the last 32 one by one (through the decode
    graph); and in portions 7, 2, 160, 3, 2, 129, with pages of 16 and of 64 tokens."""
    from aegean_tge_b200 import ops
    tokens = _tokens(shape, 303, salt=1)
    ref = _oracle(shape).logits(dtype, tokens)
    engine = _engine(shape, dtype)
    whole = _pick(engine.runner.step([_portion("w", tokens)]))
    engine.runner.finish("w")
    _close(whole, ref, dtype, f"{shape} whole prompt")
    rows = [_pick(engine.runner.step([_portion("r", tokens[:271])]))]
    for t in range(271, 303):
        rows.append(_pick(engine.runner.step([_portion("r", tokens[t:t + 1])])))
    engine.runner.finish("r")
    assert engine.runner.graph_replays >= 32
    _close(torch.cat(rows), ref, dtype, f"{shape} last 32 one by one")
    if dtype == "float32":
        assert float((torch.cat(rows) - whole).abs().max()) <= 1e-5 * float(ref.abs().max())
    del engine
    for page_size in (64, 16):
        engine = _engine(shape, dtype, page_size=page_size)
        rows, pos = [], 0
        for count in (7, 2, 160, 3, 2, 129):
            rows.append(_pick(engine.runner.step([_portion("p", tokens[pos:pos + count])])))
            pos += count
        assert pos == len(tokens)
        _close(torch.cat(rows), ref, dtype, f"{shape} portions, pages of {page_size}")
        ops.check_status()
        engine.cache.check()
        del engine


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", list(SHAPES))
@pytest.mark.parametrize("page_size,pool_tokens", [(16, 320), (64, 512)])
def test_mixed_batches_with_page_reuse(shape, dtype, page_size, pool_tokens):
    """Up to four live requests, prompt portions beside decoded tokens, so few pages that they are used again."""
    from aegean_tge_b200 import ops
    lengths = {"a": 70, "b": 45, "c": 130, "d": 19, "e": 64, "f": 33}
    tokens = {r: _tokens(shape, n, salt=ord(r)) for r, n in lengths.items()}
    engine = _engine(shape, dtype, max_tokens=pool_tokens, page_size=page_size)
    seen_pages = set()
    got = {r: [] for r in lengths}
    done = {r: 0 for r in lengths}

    def run(step):
        logits = _pick(engine.runner.step([_portion(r, tokens[r][done[r]:done[r] + count]) for r, count in step]))
        row = 0
        for r, count in step:
            got[r].append(logits[row:row + count])
            row += count
            done[r] += count
            seen_pages.update(x for x in engine.cache.groups[0].tables[r] if x >= 0)
            if done[r] == lengths[r]:
                engine.runner.finish(r)
        engine.cache.check()

    run([("a", 33)])
    run([("a", 1), ("b", 20)])
    run([("b", 2), ("a", 1), ("c", 50)])
    run([("c", 30), ("a", 1), ("b", 1), ("d", 19)])
    run([("a", 34), ("b", 22), ("c", 1)])
    run([("c", 49), ("e", 17)])
    run([("e", 2), ("f", 30)])
    run([("f", 1), ("e", 1)])
    run([("e", 44), ("f", 2)])
    total_pages = sum(-(-n // page_size) for n in lengths.values())
    assert len(seen_pages) <= engine.cache.groups[0].pool.capacity < total_pages
    oracle = _oracle(shape)
    for r in lengths:
        _close(torch.cat(got[r]), oracle.logits(dtype, tokens[r]), dtype, f"{shape} mixed, pages of {page_size}, request {r}")
    ops.check_status()
    assert all(g.pool.free_count == g.pool.capacity for g in engine.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", list(SHAPES))
def test_many_decode_rows(shape, dtype):
    """150 requests decode one token each in one step, then 64 of them one more: the widths at which the
    products change their plan (two-SM tiles above 128 rows, cuts along k, rows that travel without their
    norm factor up to 128).  The requests repeat five short sequences; the engine does not know."""
    from aegean_tge_b200 import ops
    distinct = [_tokens(shape, n, salt=50 + n) for n in (5, 7, 10, 13, 8)]
    ref = [_oracle(shape).logits(dtype, seq) for seq in distinct]
    engine = _engine(shape, dtype, max_requests=150, max_tokens=150 * 64)
    names = list(range(150))
    prompt = {r: len(distinct[r % 5]) - 2 for r in names}
    engine.runner.step([_portion(r, distinct[r % 5][:prompt[r]], []) for r in names])
    first = _pick(engine.runner.step([_portion(r, [distinct[r % 5][prompt[r]]]) for r in names]))
    want = torch.stack([ref[r % 5][prompt[r]] for r in names])
    _close(first, want, dtype, f"{shape} 150 decode rows")
    some = names[:64]
    second = _pick(engine.runner.step([_portion(r, [distinct[r % 5][prompt[r] + 1]]) for r in some]))
    want = torch.stack([ref[r % 5][prompt[r] + 1] for r in some])
    _close(second, want, dtype, f"{shape} 64 decode rows")
    ops.check_status()


def test_a_captured_graph_survives_the_growth_of_the_scratch_buffer():
    """The products' partial sums go to one scratch buffer whose address a captured decode graph holds.  A later
    prompt portion that needs a larger buffer must leave the old one alive: the graph is replayed afterwards
    and must still give what an engine without graphs gives."""
    from aegean_tge_b200 import ops
    device = torch.cuda.current_device()
    if device in ops._scratch:                       # start from the smallest buffer, as a fresh process would
        ops._outgrown.setdefault(device, []).append(ops._scratch.pop(device))
    tokens = _tokens("7B", 40, salt=9)
    # 256 tokens: the down product is cut in five along k there (few tiles, a long k), 4.6 M partial sums where the
    # first buffer holds 4 Mi; longer portions have tiles enough and are not cut
    long_prompt = _tokens("7B", 256, salt=10)
    outputs = []
    for use_graphs in (True, False):
        engine = _engine("7B", "bfloat16", use_graphs=use_graphs, run_ahead=False, max_tokens=4096)
        rows = [_pick(engine.runner.step([_portion("r", tokens[:8])]))]
        for t in range(8, 24):
            rows.append(_pick(engine.runner.step([_portion("r", tokens[t:t + 1])])))
        small = ops._scratch[device].numel()
        engine.runner.step([_portion("big", long_prompt, [])])
        if use_graphs:
            assert ops._scratch[device].numel() > small, "the long portion was meant to outgrow the scratch buffer"
            assert any(old.numel() == small for old in ops._outgrown[device])
        for t in range(24, 40):
            rows.append(_pick(engine.runner.step([_portion("r", tokens[t:t + 1])])))
        assert engine.runner.graph_replays == (32 if use_graphs else 0)
        outputs.append(torch.cat(rows))
        del engine
    ops.check_status()
    assert torch.equal(outputs[0], outputs[1])
    _close(outputs[0], _oracle("7B").logits("bfloat16", tokens), "bfloat16", "7B decode around a scratch growth")
