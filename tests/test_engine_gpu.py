"""The engine against the plain implementation: every way of cutting and batching, both dtypes."""
import random

import pytest
import torch

from conftest import TINY
from helpers import MODEL_TOL, model_tol, rel_error
from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
MODELS = ["A", "B", "C", "D", "E"]


def _tokens(name, count, salt=0):
    config, seed = TINY[name]
    rnd = random.Random(seed * 100 + salt)
    return [rnd.randrange(config["vocab_size"]) for _ in range(count)]


@pytest.fixture(scope="module")
def oracle(model_dirs):
    cache = {}

    def get(name, tokens):
        key = (name, tuple(tokens))
        if key not in cache:
            if name not in cache:
                cache[name] = plain.read_model(model_dirs[name])
            config, weights = cache[name]
            cache[key] = plain.logits_of(config, weights, tokens).float()
        return cache[key]
    return get


def _engine(model_dirs, name, dtype, **kw):
    from aegean_tge_b200 import Engine
    kw.setdefault("context", 256)
    kw.setdefault("max_tokens", 1024)
    kw.setdefault("max_requests", 8)
    return Engine(model_dirs[name], dtype=dtype, **kw)


def _portion(request, tokens, want=None):
    from aegean_tge_b200.engine import Portion
    return Portion(request, tokens, list(range(len(tokens))) if want is None else want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_whole_prompt(model_dirs, oracle, name, dtype):
    """Each request alone and whole, at several lengths including one token and page edges."""
    from aegean_tge_b200 import ops
    engine = _engine(model_dirs, name, dtype)
    for length in (1, 7, 16, 33, 130):
        tokens = _tokens(name, length, salt=length)
        logits = engine.runner.step([_portion("r", tokens)])
        engine.runner.finish("r")
        assert rel_error(logits, oracle(name, tokens)) < model_tol(dtype, name), (name, dtype, length)
    ops.check_status()
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_last_32_tokens_one_by_one(model_dirs, oracle, name, dtype):
    """Most of the sequence in one step, the last 32 tokens decoded one at a time."""
    tokens = _tokens(name, 100, salt=1)
    ref = oracle(name, tokens)
    engine = _engine(model_dirs, name, dtype)
    rows = [engine.runner.step([_portion("r", tokens[:68])])]
    for t in range(68, 100):
        rows.append(engine.runner.step([_portion("r", tokens[t:t + 1])]))
    got = torch.cat(rows)
    assert rel_error(got, ref) < model_tol(dtype, name)
    if dtype == "float32":
        # decoding a token and running it inside a prompt are the same arithmetic per row
        whole = _engine(model_dirs, name, dtype).runner.step([_portion("w", tokens)])
        assert float((got - whole).abs().max()) <= 1e-5 * float(ref.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
@pytest.mark.parametrize("page_size", [16, 64])
def test_portions_of_changing_size(model_dirs, oracle, name, dtype, page_size):
    tokens = _tokens(name, 120, salt=2)
    ref = oracle(name, tokens)
    engine = _engine(model_dirs, name, dtype, page_size=page_size)
    cuts = [7, 2, 16, 3, 2, 30, 2, 17, 41]
    assert sum(cuts) == len(tokens)
    rows, pos = [], 0
    for count in cuts:
        rows.append(engine.runner.step([_portion("r", tokens[pos:pos + count])]))
        pos += count
    assert rel_error(torch.cat(rows), ref) < model_tol(dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
@pytest.mark.parametrize("page_size,pool_tokens", [(16, 320), (64, 512), (32, 384)])
def test_mixed_batches_with_page_reuse(model_dirs, oracle, name, dtype, page_size, pool_tokens):
    """Up to four live requests, prompt portions beside decoded tokens, so few pages that they are reused."""
    from aegean_tge_b200 import ops
    lengths = {"a": 70, "b": 45, "c": 130, "d": 19, "e": 64, "f": 33}
    tokens = {r: _tokens(name, n, salt=ord(r)) for r, n in lengths.items()}
    # pages of 16: 20 pages, a+b+c+d alone need 18; of 64: 8 pages for 7; of 32: 12 pages for 11
    engine = _engine(model_dirs, name, dtype, max_tokens=pool_tokens, page_size=page_size)
    seen_pages = set()
    got = {r: [] for r in lengths}
    done = {r: 0 for r in lengths}

    def run(step):
        portions = []
        for r, count in step:
            portions.append(_portion(r, tokens[r][done[r]:done[r] + count]))
        logits = engine.runner.step(portions)
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
    run([("c", 30), ("a", 1), ("b", 1), ("d", 19)])            # d finishes: its pages go back
    run([("a", 34), ("b", 22), ("c", 1)])                      # a and b finish
    run([("c", 49), ("e", 17)])                                # c finishes; e starts on reused pages
    run([("e", 2), ("f", 30)])
    run([("f", 1), ("e", 1)])
    run([("e", 44), ("f", 2)])
    assert all(done[r] == lengths[r] for r in lengths)
    total_pages = sum(-(-n // page_size) for n in lengths.values())
    assert len(seen_pages) <= engine.cache.groups[0].pool.capacity < total_pages       # pages were used again
    for r in lengths:
        assert rel_error(torch.cat(got[r]), oracle(name, tokens[r])) < model_tol(dtype, name), r
    ops.check_status()
    assert not engine.cache.live_requests()
    assert all(g.pool.free_count == g.pool.capacity for g in engine.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page_size", [16, 64])
def test_long_decoding(model_dirs, oracle, dtype, page_size):
    """A short prompt, then 200 tokens one by one (teacher-forced), across many page edges."""
    name = "B"
    tokens = _tokens(name, 210, salt=3)
    ref = oracle(name, tokens)
    engine = _engine(model_dirs, name, dtype, page_size=page_size)
    rows = [engine.runner.step([_portion("r", tokens[:10])])]
    for t in range(10, 210):
        rows.append(engine.runner.step([_portion("r", tokens[t:t + 1])]))
    assert rel_error(torch.cat(rows), ref) < model_tol(dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_first_tokens_of_a_sequence(model_dirs, oracle, name, dtype):
    """Positions 0, 1, 2: one key, the first rotation angles, a page with one slot in use."""
    tokens = _tokens(name, 3, salt=4)
    ref = oracle(name, tokens)
    engine = _engine(model_dirs, name, dtype)
    rows = [engine.runner.step([_portion("r", tokens[t:t + 1])]) for t in range(3)]
    assert rel_error(torch.cat(rows), ref) < model_tol(dtype, name)


def test_only_wanted_rows_come_back(model_dirs, oracle):
    tokens = _tokens("A", 40, salt=5)
    ref = oracle("A", tokens)
    engine = _engine(model_dirs, "A", "float32")
    assert engine.runner.step([_portion("r", tokens[:20], want=[])]) is None
    logits = engine.runner.step([_portion("r", tokens[20:], want=[19, 0])])
    assert logits.shape == (2, 256)
    assert rel_error(logits, ref[[39, 20]]) < MODEL_TOL["float32"]


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(model_dirs, dtype):
    """Engine.generate against the plain implementation's greedy continuation (float32: token for token)."""
    from aegean_tge_b200 import Engine
    name = "B"
    config, weights = plain.read_model(model_dirs[name])
    prompts = [_tokens(name, n, salt=50 + n) for n in (1, 7, 33)]
    engine = Engine(model_dirs[name], dtype=dtype, context=128, max_tokens=512, max_batch_tokens=16, max_requests=4)
    outputs = engine.generate(prompts, n=16)
    for prompt, output in zip(prompts, outputs):
        assert len(output) == 16
        if dtype == "float32":
            assert output == plain.greedy(config, weights, prompt, 16)
        else:
            # bfloat16 may flip a near-tie: every chosen token must be within tolerance of the best one
            tokens = list(prompt)
            for token in output:
                row = plain.logits_of(config, weights, tokens)[-1]
                assert float(row.max() - row[token]) < model_tol(dtype, name) * float(row.abs().max())
                tokens.append(token)
    single = engine.generate(prompts[1], n=4)
    assert single == outputs[1][:4]


def test_generation_does_not_depend_on_pages_or_budget(model_dirs):
    """Same requests, same tokens, whatever the pool size, token budget and chunk (preemption included)."""
    from aegean_tge_b200 import Engine, SamplingParams
    name = "A"
    prompts = [_tokens(name, n, salt=70 + n) for n in (5, 19, 64, 130)]
    params = [SamplingParams(temperature=0.8, seed=11 + i) for i in range(4)]
    outputs = []
    for kw in (dict(max_tokens=2048, max_batch_tokens=512, run_ahead=False),
               dict(max_tokens=2048, max_batch_tokens=512), dict(max_tokens=2048, max_batch_tokens=16, chunk=16),
               dict(num_pages=15, page_size=16, max_batch_tokens=16, chunk=16),
               dict(num_pages=13, page_size=16, max_batch_tokens=40, chunk=7),
               dict(num_pages=5, page_size=64, max_batch_tokens=40, chunk=24),
               dict(num_pages=7, page_size=32, max_batch_tokens=16)):
        engine = Engine(model_dirs[name], dtype="float32", context=256, max_requests=4, **kw)
        outputs.append(engine.generate(prompts, n=24, sampling=params))
        engine.cache.check()
        assert all(g.pool.free_count == g.pool.capacity for g in engine.cache.groups)
        if "num_pages" in kw:
            assert engine.stats()["preemptions"] > 0
    assert all(o == outputs[0] for o in outputs[1:])


def test_sampled_generation_is_the_plain_samplers_walk(model_dirs):
    """Tiny B, four requests with prompts of 5, 19, 64 and 130 tokens, prompts in portions of 16 beside decode
    steps, 24 tokens each at temperature 0.8 from per-request seeds: the expected tokens come from the plain
    model and the plain sampler walking each request's xorshift32 stream token by token on the CPU
    (src/models/sampling.cpp:183-228, :72-93, :16-28), for every pool, budget and chunk (preemption included).
    The kernel sums the probabilities in segments, the plain walk one by one, so a draw that lands within
    vocab * 2^-24 of a boundary between two tokens may fall on either side: at most one such token is let
    through, and only if the draw really lies that close."""
    import numpy as np
    from aegean_tge_b200 import Engine, SamplingParams
    name, temperature, count = "B", 0.8, 24
    config, weights = plain.read_model(model_dirs[name])
    vocab = config["vocab_size"]
    prompts = [_tokens(name, n, salt=70 + n) for n in (5, 19, 64, 130)]
    params = [SamplingParams(temperature=temperature, seed=11 + i) for i in range(4)]
    outputs = []
    for kw in (dict(max_tokens=2048, max_batch_tokens=16, chunk=16), dict(max_tokens=2048, max_batch_tokens=512, run_ahead=False),
               dict(max_tokens=2048, max_batch_tokens=512), dict(num_pages=15, page_size=16, max_batch_tokens=16, chunk=16),
               dict(num_pages=13, page_size=16, max_batch_tokens=40, chunk=7),
               dict(num_pages=5, page_size=64, max_batch_tokens=40, chunk=24)):
        engine = Engine(model_dirs[name], dtype="float32", context=256, max_requests=4, **kw)
        outputs.append(engine.generate(prompts, n=count, sampling=params))
        engine.cache.check()
        if "num_pages" in kw:
            assert engine.stats()["preemptions"] > 0
    assert all(o == outputs[0] for o in outputs[1:])
    close_calls = 0
    for prompt, param, got in zip(prompts, params, outputs[0]):
        rng = plain.PlainXorShift32(param.seed)
        tokens = list(prompt)
        assert len(got) == count
        for token in got:
            row = plain.logits_of(config, weights, tokens)[-1].float().numpy()
            state = rng.state
            expected = plain.sample_plain(row, temperature, rng)
            if token != expected:
                # the same draw against the exact cumulative sums: it must lie at the boundary between the two tokens
                replay = plain.PlainXorShift32(1)
                replay.state = state
                p = np.exp((row.astype(np.float64) - float(row.max())) / temperature)
                target = float(replay.next()) * p.sum()
                edges = np.cumsum(p)
                lo, hi = sorted((token, expected))
                assert hi == lo + 1 or float(p[lo + 1:hi].sum()) < vocab * 2.0 ** -24 * p.sum(), (token, expected)
                assert abs(target - edges[lo]) < vocab * 2.0 ** -24 * p.sum(), (token, expected, target, edges[lo])
                close_calls += 1
            tokens.append(token)
    assert close_calls <= 1


@pytest.mark.parametrize("name", ["B", "D"])
def test_many_requests_in_one_step(model_dirs, oracle, name):
    """150 requests at once in bfloat16: their prompts in one step (450 rows) and then one decoded token each
    (150 rows, a replayed graph), sizes at which the products pair two SMs on a tile and cut along k."""
    from aegean_tge_b200 import ops
    count = 150
    engine = _engine(model_dirs, name, "bfloat16", max_tokens=count * 64, max_requests=count, max_batch_tokens=512)
    prompts = [_tokens(name, 3, salt=1000 + i) for i in range(count)]
    nexts = [_tokens(name, 1, salt=5000 + i) for i in range(count)]
    first = engine.runner.step([_portion(f"r{i}", prompts[i], [2]) for i in range(count)])
    for repeat in range(2):      # the second decode step replays the graph the first one captured or warmed
        second = engine.runner.step([_portion(f"r{i}", nexts[i] if repeat == 0 else [7], [0]) for i in range(count)])
        if repeat == 0:
            kept = second.clone()
    assert first.shape[0] == count and kept.shape[0] == count
    for i in (0, 1, 63, 64, 127, 128, 149):
        assert rel_error(first[i], oracle(name, prompts[i])[2]) < model_tol("bfloat16", name), (name, i)
        assert rel_error(kept[i], oracle(name, prompts[i] + nexts[i])[3]) < model_tol("bfloat16", name), (name, i)
        assert rel_error(second[i], oracle(name, prompts[i] + nexts[i] + [7])[4]) < model_tol("bfloat16", name), (name, i)
    ops.check_status()
    for i in range(count):
        engine.runner.finish(f"r{i}")
    engine.cache.check()


def test_kernels_are_loaded_and_cpu_is_refused(model_dirs):
    from aegean_tge_b200 import ops
    _engine(model_dirs, "A", "bfloat16")
    names = " ".join(ops.loaded_libraries())
    assert "libtge_core.so" in names and "libtge_attn_hd16.so" in names
    with pytest.raises(ops.KernelError):
        ops.rmsnorm(torch.zeros(2, 8), torch.ones(8), 1e-6, torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_context_in_portions_then_decoding(model_dirs, oracle, dtype):
    """1,500 positions: prompt portions of 600 (several key splits and page-table staging), then tokens one by one."""
    name = "D"
    tokens = _tokens(name, 1500, salt=9)
    ref = oracle(name, tokens)
    engine = _engine(model_dirs, name, dtype, context=2048, max_tokens=2048)
    rows = []
    for begin in (0, 600, 1200):
        count = min(600, 1480 - begin)
        rows.append(engine.runner.step([_portion("r", tokens[begin:begin + count], want=[count - 1])]))
    for t in range(1480, 1500):
        rows.append(engine.runner.step([_portion("r", tokens[t:t + 1])]))
    got = torch.cat(rows)
    want = ref[[599, 1199, 1479] + list(range(1480, 1500))]
    assert rel_error(got, want) < model_tol(dtype, name)


def test_tensor_core_and_cuda_core_paths_agree_at_a_large_layer_shape():
    """A two-layer model with the layer sizes of a 14B model (hidden 5120, 40 heads on 8 kv heads of 128,
    feed-forward 13824): bfloat16 logits through the tcgen05/TMA kernels against the CUDA-core kernels."""
    from aegean_tge_b200 import Engine, ops
    config = {"architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 5120,
              "num_attention_heads": 40, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 13824,
              "vocab_size": 3000, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
              "max_position_embeddings": 1024}
    rnd = random.Random(4)
    tokens = [rnd.randrange(3000) for _ in range(300)]
    engine = Engine(random_config=config, seed=5, dtype="bfloat16", context=512, max_tokens=1024, max_requests=4)

    def run():
        out = [engine.runner.step([_portion("r", tokens[:280], want=[279, 0])])]
        for t in range(280, 300):
            out.append(engine.runner.step([_portion("r", tokens[t:t + 1])]))
        engine.runner.finish("r")
        return torch.cat(out).float().cpu()
    fast = run()
    ops.USE_TCGEN05, ops.USE_MMA_ATTENTION = False, False
    engine.runner.use_graphs = False            # a captured graph would replay the kernels it was captured with
    try:
        slow = run()
    finally:
        ops.USE_TCGEN05, ops.USE_MMA_ATTENTION = True, True
    ops.check_status()
    assert rel_error(fast, slow) < MODEL_TOL["bfloat16"]


def test_bench_continuous_transcripts_are_identical(model_dirs, capsys):
    """The reference's leak check (apps/cli/main.cpp:1620-1643): every request gets the same prompt, more
    requests than slots, so requests start beside others at every stage; in float32 all transcripts are equal."""
    from aegean_tge_b200.cli import main
    code = main(["bench", "continuous", "--model", model_dirs["B"], "--dtype", "float32", "--requests", "7",
                 "--sequences", "3", "--tokens", "12", "--prompt-tokens", "21", "--context", "128", "--num-pages", "9",
                 "--page-size", "16", "--max-batch-tokens", "16"])
    out = capsys.readouterr().out
    assert code == 0, out
    assert "independent (all transcripts identical)" in out and "7 requests, 3 slots" in out
    code = main(["bench", "continuous", "--model", model_dirs["A"], "--requests", "5", "--sequences", "2", "--tokens", "6",
                 "--prompt-tokens", "3", "--prompt-max", "40", "--context", "128"])
    assert code == 0 and "not compared" in capsys.readouterr().out


def test_fidelity_of_the_bfloat16_kernels(model_dirs, capsys):
    """`tge fidelity`: the float32 path as oracle, the bfloat16 kernels as candidate, teacher-forced."""
    import re
    from aegean_tge_b200.cli import main
    assert main(["fidelity", "--model", model_dirs["B"], "--tokens", "90", "--context", "128"]) == 0
    out = capsys.readouterr().out
    mean_kl = float(re.search(r"KL       : mean ([0-9.e+-]+)", out).group(1))
    agree, total = map(int, re.search(r"top-1    : (\d+)/(\d+) agree", out).groups())
    assert total == 90 and mean_kl < 1e-3 and agree >= 80, out


def test_steps_queued_ahead_change_nothing(model_dirs, tmp_path):
    """Decode steps are queued before the previous step's tokens are read.  With and without that the same
    tokens come out: greedy and temperature rows, requests of different lengths, and a request that ends on an
    end token (the step queued for it is dropped and its generator put back)."""
    import json
    import shutil
    from aegean_tge_b200 import Engine, SamplingParams
    prompts = [_tokens("A", n, salt=90 + n) for n in (9, 30, 17)]
    params = [SamplingParams(temperature=0.9, seed=5), SamplingParams(), SamplingParams(temperature=0.7, seed=6)]

    def run(folder, run_ahead):
        engine = Engine(folder, dtype="float32", context=256, max_tokens=1024, max_requests=4, run_ahead=run_ahead)
        ids = [engine.add_request(p, n, s) for p, n, s in zip(prompts, (40, 25, 33), params)]
        done = {}
        while engine.has_unfinished():
            for request in engine.step():
                done[request.id] = request
        engine.cache.check()
        return [done[i].output for i in ids], [done[i].finish_reason for i in ids], engine.stats()["steps_queued_ahead"]

    plain, reasons, counts = run(model_dirs["A"], False)
    assert counts == {"used": 0, "dropped": 0} and reasons == ["length"] * 3
    ahead, _, counts = run(model_dirs["A"], True)
    assert ahead == plain and counts["used"] > 20
    # the same model with an end token that the first request draws on its way
    stop = plain[0][15]
    folder = tmp_path / "with_end_token"
    shutil.copytree(model_dirs["A"], folder)
    config = json.loads((folder / "config.json").read_text())
    config["eos_token_id"] = stop
    (folder / "config.json").write_text(json.dumps(config))
    plain, reasons, _ = run(str(folder), False)
    assert "end_token" in reasons
    ahead, reasons_ahead, counts = run(str(folder), True)
    assert ahead == plain and reasons_ahead == reasons and counts["dropped"] >= 1 and counts["used"] > 5


def test_decode_graphs_are_capped_and_share_a_pool(model_dirs, oracle):
    """Decode steps at several batch sizes capture a graph for each size class (1, 2, 4, ...); only the most
    recently used ones are kept, they allocate from one pool, and a graph that was dropped is simply captured
    again: the logits stay those of the plain model whichever graphs live."""
    name, dtype = "D", "float32"
    engine = _engine(model_dirs, name, dtype, max_requests=6)
    engine.runner.max_graphs = 2
    prompts = [_tokens(name, 6 + i, salt=300 + i) for i in range(5)]
    nexts = [_tokens(name, 6, salt=400 + i) for i in range(5)]
    engine.runner.step([_portion(i, prompts[i], []) for i in range(5)])
    done = [0] * 5
    for batch in (1, 2, 3, 1, 4, 2):                              # 3 and 4 share a graph; 1 and 2 come back after they were dropped
        rows = engine.runner.step([_portion(i, [nexts[i][done[i]]]) for i in range(batch)])
        for i in range(batch):
            done[i] += 1
            ref = oracle(name, prompts[i] + nexts[i][:done[i]])[-1]
            assert rel_error(rows[i], ref) < model_tol(dtype, name), (batch, i)
        assert len(engine.runner._graphs) <= 2
    assert engine.runner.graphs_captured == 5 and engine.runner.graph_replays == 6
    assert engine.runner._graph_pool is not None


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_graphs_serve_a_range_of_batch_sizes_with_idle_rows(model_dirs, oracle, dtype):
    """Above eight rows a decode graph is captured for the next of a few sizes and smaller batches run it with
    idle rows behind the real ones (one token on the scratch page, state in the scratch slot).  The real rows'
    logits are the plain model's, the idle rows leave nothing behind in the pages that requests hold, and a
    batch that shrinks from 12 to 9 keeps replaying one graph."""
    from aegean_tge_b200.engine.runner import graph_batch
    assert [graph_batch(b) for b in (1, 2, 3, 4, 5, 8, 9, 12, 13, 16, 17, 25, 33, 49, 64, 65, 200)] == \
        [1, 2, 4, 4, 8, 8, 12, 12, 16, 16, 24, 32, 48, 64, 64, 96, 256]
    name = "E"
    engine = _engine(model_dirs, name, dtype, max_requests=13)
    count = 12
    prompts = [_tokens(name, 5 + 3 * i, salt=500 + i) for i in range(count)]
    nexts = [_tokens(name, 5, salt=600 + i) for i in range(count)]
    engine.runner.step([_portion(i, prompts[i], []) for i in range(count)])
    done = [0] * count
    for batch in (12, 11, 10, 9, 13):
        if batch == 13:                                           # one more request joins: the next size's graph
            prompts.append(_tokens(name, 7, salt=700))
            nexts.append(_tokens(name, 5, salt=701))
            done.append(0)
            engine.runner.step([_portion(12, prompts[12], [])])
        rows = engine.runner.step([_portion(i, [nexts[i][done[i]]]) for i in range(batch)])
        assert rows.shape[0] == batch
        for i in range(batch):
            done[i] += 1
            ref = oracle(name, prompts[i] + nexts[i][:done[i]])[-1]
            assert rel_error(rows[i], ref) < model_tol(dtype, name), (batch, i)
    assert engine.runner.graphs_captured == 2 and engine.runner.graph_replays == 5
    assert sorted(key[0] for key in engine.runner._graphs) == [12, 16]
    engine.cache.check()


@pytest.mark.parametrize("max_tokens,preempts", [(4096, False), (192, True)])
def test_many_requests_with_every_sampler_finish_and_give_their_pages_back(model_dirs, max_tokens, preempts):
    """Forty requests of mixed lengths, greedy, temperature, top-k/top-p and min-p with a repetition penalty, through
    twelve slots: with room for all, and with so few pages that requests are preempted and start over.  Everyone
    gets exactly the tokens asked for, every page and slot comes back, no kernel reported a fault."""
    from aegean_tge_b200 import SamplingParams, ops
    name = "D"
    engine = _engine(model_dirs, name, "bfloat16", context=128, max_tokens=max_tokens, max_requests=12, page_size=16,
                     max_batch_tokens=96)
    rnd = random.Random(11)
    vocab = TINY[name][0]["vocab_size"]
    want = {}
    for i in range(40):
        prompt = [rnd.randrange(vocab) for _ in range(rnd.randint(5, 60))]
        sampling = [None, SamplingParams(temperature=0.9, seed=i + 1),
                    SamplingParams(temperature=0.8, top_k=10, top_p=0.9, seed=i + 1),
                    SamplingParams(temperature=1.0, min_p=0.05, repeat_penalty=1.1, seed=i + 1)][i % 4]
        count = rnd.randint(3, 40)
        want[engine.add_request(prompt, count, sampling)] = count
    lengths = want
    done = {}
    while engine.has_unfinished():
        for request in engine.step():
            done[request.id] = request
    ops.check_status()
    engine.cache.check()
    assert set(done) == set(want)
    assert all(len(done[i].output) == lengths[i] for i in want)
    assert all(0 <= t < vocab for r in done.values() for t in r.output)
    stats = engine.stats()
    assert (stats["preemptions"] > 0) == preempts
    assert all(g["free"] == g["capacity"] for g in stats["pages"])


def test_command_line_generates_and_benches(model_dirs, capsys):
    """`tge generate` and the three single-step benches on a tiny model: exit codes and the labels of their lines."""
    from aegean_tge_b200.cli import main
    assert main(["generate", "--model", model_dirs["D"], "--tokens", "5 17 3", "--n", "6", "--print-ids", "--context", "128"]) == 0
    out = capsys.readouterr().out
    assert "prefill  :" in out and "decode   :" in out and len(out.split("ids      :")[1].split()) == 6
    common = ["--model", model_dirs["D"], "--context", "512", "--max-requests", "12", "--page-size", "16"]
    assert main(["bench", "decode", *common, "--batch", "3", "--prompt-len", "40", "--n", "4"]) == 0
    assert main(["bench", "prefill", *common, "--prompt-len", "100", "--repeat", "1"]) == 0
    assert main(["bench", "mixed", *common, "--batch", "9", "--prompt-len", "40", "--portion", "70", "--timeline"]) == 0
    out = capsys.readouterr().out
    assert "decode   : batch 3 at context 40" in out and "after a pause" in out
    assert "mixed    : 9 single tokens at context 40 beside a portion of 70 tokens" in out
    assert "attention_decode" in out and "span of the step" in out           # the nine single tokens took the decode kernel
