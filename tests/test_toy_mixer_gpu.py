"""A mixer with state of its own, defined here, registered, built and stepped through the engine
without touching the package: the layer list mixes it with attention, and a second toy
architecture runs a layer twice and lets a layer read another layer's cache."""
import random

import pytest
import torch

from helpers import MODEL_TOL, rel_error
from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

HIDDEN, VOCAB, HEADS, KV, HD, INNER = 48, 97, 3, 1, 16, 80


def _register():
    from aegean_tge_b200.config.model_spec import LayerSpec, ModelSpec, PartSpec
    from aegean_tge_b200.parts.base import MIXERS, Mixer, ParamSpec, StateSpec
    from aegean_tge_b200.registry import Architecture, register_architecture, registered_architectures
    from aegean_tge_b200.weights import normal, uniform

    if "toy_running_mean" not in MIXERS.names():
        @MIXERS.register("toy_running_mean")
        class RunningMean(Mixer):
            """y_t = W mean(h_0..h_t): the running sum and the count live in the request's state slot."""

            def __init__(self, spec, env):
                super().__init__(spec, env)
                self.hidden = int(spec.params["hidden_size"])
                self.weight = None

            def param_specs(self):
                return {"mix.weight": ParamSpec((self.hidden, self.hidden))}

            def load(self, tensors):
                self.weight = tensors["mix.weight"]

            def state_spec(self):
                return StateSpec((("sum", (self.hidden,)), ("count", (1,))))

            def flops(self, tokens, pairs):
                return 2.0 * tokens * self.hidden * self.hidden

            def forward(self, h, ctx, cache):
                out = torch.empty_like(h)
                begin = 0
                for count, slot in zip(ctx.host_q_lens, ctx.host_slots):
                    part = h[begin:begin + count].float()
                    running = cache.state["sum"][slot] + torch.cumsum(part, dim=0)
                    seen = cache.state["count"][slot] + torch.arange(1, count + 1, device=h.device)[:, None]
                    cache.state["sum"][slot] = running[-1]
                    cache.state["count"][slot] += count
                    out[begin:begin + count] = ((running / seen) @ self.weight.float().T).to(h.dtype)
                    begin += count
                return out

    if "toy_running_mean_on_device" not in MIXERS.names():
        @MIXERS.register("toy_running_mean_on_device")
        class RunningMeanOnDevice(MIXERS.get("toy_running_mean")):
            """The same mixer working from the step's device arrays only (``ctx.slots``, ``ctx.q_start``): no host
            lists, no synchronisation, so single-token steps may be replayed from a CUDA graph and queued ahead."""
            graph_safe = True

            def forward(self, h, ctx, cache):
                seq, slots = ctx.seq_of_token.long(), ctx.slots.long()
                part = h.float()
                summed = torch.cumsum(part, dim=0)
                first = ctx.q_start[:-1].long()
                before = summed[first] - part[first]                      # the sum of everything before each portion
                running = cache.state["sum"][slots][seq] + (summed - before[seq])
                seen = (ctx.positions + 1).float()[:, None]                # tokens of the request up to and with this one
                last = ctx.q_start[1:].long() - 1
                cache.state["sum"].index_copy_(0, slots, running[last])
                cache.state["count"].index_copy_(0, slots, seen[last])
                return ((running / seen) @ self.weight.float().T).to(h.dtype)

    def build_spec(config):
        position = PartSpec("rope_neox", {"head_dim": HD, "theta": 777.0})
        norm = lambda name: PartSpec("rmsnorm", {"size": HIDDEN, "eps": 1e-5}, {"weight": name})
        layers = []
        for n, kind in enumerate(config["kinds"]):
            p = f"layers.{n}."
            if kind in ("toy", "toy_on_device"):
                mixer = PartSpec("toy_running_mean" if kind == "toy" else "toy_running_mean_on_device",
                                 {"hidden_size": HIDDEN}, {"mix.weight": p + "mix.weight"})
            else:
                mixer = PartSpec("gqa_attention",
                                 {"hidden_size": HIDDEN, "heads": HEADS, "kv_heads": KV, "head_dim": HD,
                                  "qkv_bias": kind == "attention_bias", "o_bias": False,
                                  "window": config.get("window") if kind == "attention_window" else None,
                                  "position": position},
                                 {f"{x}.{y}": p + f"{x}.{y}" for x in "qkvo" for y in ("weight", "bias")})
            ffn = PartSpec("swiglu", {"hidden_size": HIDDEN, "intermediate_size": INNER},
                           {f"{x}.weight": p + f"{x}.weight" for x in ("gate", "up", "down")})
            layers.append(LayerSpec("pre_norm", mixer, ffn, norm(p + "norm1"), norm(p + "norm2"),
                                    cache_from=config.get("cache_from", {}).get(n)))
        sizes = {"vocab_size": VOCAB, "hidden_size": HIDDEN}
        return ModelSpec("ToyForTests", HIDDEN, VOCAB, 256, tuple(layers), tuple(config["schedule"]),
                         PartSpec("token_embedding", sizes, {"weight": "embed"}), norm("final_norm"),
                         PartSpec("linear_head", sizes, {"weight": "head"}),
                         end_token_ids=tuple(config.get("end_token_ids", ())))

    def random_plan(config):
        def mat(*shape):
            return tuple(shape), "matrix", normal(0.08)
        def vec(n, around=0.0):
            return (n,), "vector", (uniform(around - 0.08, around + 0.08) if around else normal(0.05))
        yield ("embed", *mat(VOCAB, HIDDEN))
        yield ("head", *mat(VOCAB, HIDDEN))
        yield ("final_norm", *vec(HIDDEN, 1.0))
        for n, kind in enumerate(config["kinds"]):
            p = f"layers.{n}."
            yield (p + "norm1", *vec(HIDDEN, 1.0))
            yield (p + "norm2", *vec(HIDDEN, 1.0))
            if kind in ("toy", "toy_on_device"):
                yield (p + "mix.weight", *mat(HIDDEN, HIDDEN))
            else:
                yield (p + "q.weight", *mat(HEADS * HD, HIDDEN))
                yield (p + "k.weight", *mat(KV * HD, HIDDEN))
                yield (p + "v.weight", *mat(KV * HD, HIDDEN))
                yield (p + "o.weight", *mat(HIDDEN, HEADS * HD))
                if kind == "attention_bias":
                    yield (p + "q.bias", *vec(HEADS * HD))
                    yield (p + "k.bias", *vec(KV * HD))
                    yield (p + "v.bias", *vec(KV * HD))
            for x, shape in (("gate", (INNER, HIDDEN)), ("up", (INNER, HIDDEN)), ("down", (HIDDEN, INNER))):
                yield (p + f"{x}.weight", *mat(*shape))

    if "ToyForTests" not in registered_architectures():
        register_architecture(Architecture("ToyForTests", parse_config=lambda raw: raw, build_spec=build_spec,
                                           random_plan=random_plan))


def _plain_logits(config, w, tokens):
    """The toy architecture restated on whole sequences in float64, from the plain parts."""
    T = len(tokens)
    cos, sin = plain.rope_tables(777.0, HD, T)
    x = plain.embed(w["embed"], tokens)
    kv_of = {}
    for n in config["schedule"]:
        kind = config["kinds"][n]
        p = f"layers.{n}."
        h = plain.rms_norm(x, w[p + "norm1"], 1e-5)
        if kind in ("toy", "toy_on_device"):
            mean = torch.cumsum(h, 0) / torch.arange(1, T + 1, dtype=h.dtype)[:, None]
            x = x + mean @ w[p + "mix.weight"].T
        else:
            bias = lambda name, width: w.get(p + name, torch.zeros(width, dtype=h.dtype))
            q = plain.apply_rope((h @ w[p + "q.weight"].T + bias("q.bias", HEADS * HD)).view(T, HEADS, HD), cos, sin)
            source = config.get("cache_from", {}).get(n)
            if source is None:
                k = plain.apply_rope((h @ w[p + "k.weight"].T + bias("k.bias", KV * HD)).view(T, KV, HD), cos, sin)
                v = (h @ w[p + "v.weight"].T + bias("v.bias", KV * HD)).view(T, KV, HD)
                kv_of[n] = (k, v)
            else:
                k, v = kv_of[source]
            window = config.get("window", 0) if kind == "attention_window" else 0
            a = plain.attention(q, k, v, window=window).reshape(T, HEADS * HD)
            x = x + a @ w[p + "o.weight"].T
        h = plain.rms_norm(x, w[p + "norm2"], 1e-5)
        x = x + plain.swiglu(h, w[p + "gate.weight"], w[p + "up.weight"], w[p + "down.weight"])
    return (plain.rms_norm(x, w["final_norm"], 1e-5) @ w["head"].T).float()


def _engine_and_weights(config, dtype):
    from aegean_tge_b200 import Engine
    _register()
    raw = dict(config, architectures=["ToyForTests"])
    engine = Engine(random_config=raw, seed=3, dtype=dtype, context=256, max_tokens=512, max_requests=4)
    # read the weights back from the parts, so the oracle sees exactly what the engine holds
    w = {}
    model = engine.model
    w["embed"] = model.embedding.weight.double().cpu()
    w["head"] = model.head.weight.double().cpu()
    w["final_norm"] = model.final_norm.weight.double().cpu()
    for n, block in enumerate(model.blocks):
        p = f"layers.{n}."
        w[p + "norm1"] = block.mixer_norm.weight.double().cpu()
        w[p + "norm2"] = block.ffn_norm.weight.double().cpu()
        if config["kinds"][n] in ("toy", "toy_on_device"):
            w[p + "mix.weight"] = block.mixer.weight.double().cpu()
        else:
            qkv = block.mixer.w_qkv.double().cpu()
            w[p + "q.weight"], w[p + "k.weight"], w[p + "v.weight"] = qkv.split([HEADS * HD, KV * HD, KV * HD])
            w[p + "o.weight"] = block.mixer.w_o.double().cpu()
            if block.mixer.b_qkv is not None:
                b = block.mixer.b_qkv.double().cpu()
                w[p + "q.bias"], w[p + "k.bias"], w[p + "v.bias"] = b.split([HEADS * HD, KV * HD, KV * HD])
        gu = block.feed_forward.w_gate_up.double().cpu()
        w[p + "gate.weight"], w[p + "up.weight"] = gu[0::2], gu[1::2]
        w[p + "down.weight"] = block.feed_forward.w_down.double().cpu()
    return engine, w


CONFIGS = {
    "state_and_attention": {"kinds": ["toy", "attention_bias", "toy"], "schedule": [0, 1, 2]},
    "twice_shared_window": {"kinds": ["attention", "attention_window", "attention", "toy"], "window": 24,
                            "schedule": [0, 1, 2, 3, 1], "cache_from": {2: 0}},
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", list(CONFIGS))
def test_toy_parts_step_through_the_engine(which, dtype):
    from aegean_tge_b200.engine import Portion
    config = CONFIGS[which]
    if which == "twice_shared_window":
        # a layer that runs twice would write its cache twice; the toy keeps that layer stateless per visit
        config = dict(config, schedule=[0, 1, 2, 3])
    engine, w = _engine_and_weights(config, dtype)
    rnd = random.Random(5)
    a = [rnd.randrange(VOCAB) for _ in range(90)]
    b = [rnd.randrange(VOCAB) for _ in range(41)]
    ref_a, ref_b = _plain_logits(config, w, a), _plain_logits(config, w, b)
    full = lambda r, t: Portion(r, t, list(range(len(t))))
    got_a, got_b = [], []
    got_a.append(engine.runner.step([full("a", a[:37])]))
    out = engine.runner.step([full("a", a[37:38]), full("b", b[:20])])
    got_a.append(out[:1]); got_b.append(out[1:])
    out = engine.runner.step([full("b", b[20:22]), full("a", a[38:88])])
    got_b.append(out[:2]); got_a.append(out[2:])
    out = engine.runner.step([full("a", a[88:]), full("b", b[22:])])
    got_a.append(out[:2]); got_b.append(out[2:])
    assert rel_error(torch.cat(got_a), ref_a) < MODEL_TOL[dtype]
    assert rel_error(torch.cat(got_b), ref_b) < MODEL_TOL[dtype]
    if which == "twice_shared_window":
        assert len(engine.cache.groups) == 2                 # full-attention layers and the windowed one
        windowed = [g for g in engine.cache.groups if g.spec.window == 24][0]
        assert -1 in windowed.tables["a"]                     # pages behind the window went back
    engine.runner.finish("a"); engine.runner.finish("b")
    engine.cache.check()
    assert engine.cache.free_slots == 4


def test_a_layer_may_run_twice():
    """schedule names layer 0 (the stateful toy) twice: both visits share its weights and its state."""
    from aegean_tge_b200.engine import Portion
    config = {"kinds": ["toy", "attention"], "schedule": [0, 1, 0]}
    engine, w = _engine_and_weights(config, "float32")
    tokens = [3, 50, 7, 7, 96, 0, 12]
    logits = engine.runner.step([Portion("r", tokens, list(range(len(tokens))))])
    assert logits.shape == (len(tokens), VOCAB) and torch.isfinite(logits).all()
    assert engine.model.step_param_bytes() > 0


def _generate_with_arrivals(config, end_tokens, **engine_kw):
    """Three requests drawn at temperature 1 (the sampler stays on the device); the second and third arrive
    while the first is decoding.  Returns ({request: tokens}, engine)."""
    from aegean_tge_b200 import Engine, SamplingParams
    _register()
    raw = dict(config, architectures=["ToyForTests"], end_token_ids=list(end_tokens))
    engine = Engine(random_config=raw, seed=3, dtype="float32", context=256, max_tokens=1024, max_requests=4, **engine_kw)
    rnd = random.Random(11)
    prompts = {name: [rnd.randrange(VOCAB) for _ in range(n)] for name, n in (("a", 9), ("b", 21), ("c", 5))}
    sampling = lambda seed: SamplingParams(temperature=1.0, seed=seed)
    engine.add_request(prompts["a"], n=40, sampling=sampling(1), request_id="a")
    outputs, steps = {}, 0
    while engine.has_unfinished():
        for request in engine.step():
            outputs[request.id] = list(request.output)
        steps += 1
        if steps == 6:          # "a" decodes alone from slot 0 (its batch-1 graph exists) when "b" arrives
            engine.add_request(prompts["b"], n=30, sampling=sampling(2), request_id="b")
        if steps == 15:
            engine.add_request(prompts["c"], n=12, sampling=sampling(3), request_id="c")
    return outputs, engine


def test_state_is_safe_under_steps_queued_ahead_and_graph_capture():
    """A graph-safe mixer that updates its state slot in place.  A step queued ahead and then dropped (a request
    ended on an end token, a request arrived) must not have advanced the state, and capturing a decode graph
    for a new batch size while a request lives in slot 0 must not touch slot 0: the tokens are those of an
    engine that neither queues ahead nor replays graphs, and the last logits agree with the plain model."""
    config = {"kinds": ["toy_on_device", "attention_bias", "toy_on_device"], "schedule": [0, 1, 2]}
    free_run, _ = _generate_with_arrivals(config, (), run_ahead=False, use_graphs=False)
    # an end token that cuts at least one request short, but none before its fourth token
    end = None
    for token in range(VOCAB):
        firsts = [out.index(token) for out in free_run.values() if token in out]
        if firsts and min(firsts) >= 3 and any(token in out[:-3] for out in free_run.values()):
            end = token
            break
    assert end is not None
    plain_run, plain_engine = _generate_with_arrivals(config, (end,), run_ahead=False, use_graphs=False)
    fast_run, fast_engine = _generate_with_arrivals(config, (end,))
    assert any(out[-1] == end and len(out) < n for out, n in ((plain_run["a"], 40), (plain_run["b"], 30), (plain_run["c"], 12)))
    assert fast_run == plain_run
    stats = fast_engine.stats()["steps_queued_ahead"]
    assert stats["used"] > 0 and stats["dropped"] > 0, stats
    assert fast_engine.runner.graphs_captured >= 2 and fast_engine.runner.graph_replays > 0
    assert plain_engine.runner.graph_replays == 0 and plain_engine.stats()["steps_queued_ahead"]["used"] == 0


def test_the_host_asks_the_model_not_the_architecture(tmp_path, capsys):
    """``tge plan`` and the flop count behind ``tge bench prefill`` work for an architecture the package has
    never heard of: bytes come from the parts' declared parameters and cache needs, operations from ``flops``."""
    import json
    from aegean_tge_b200 import cli
    from aegean_tge_b200.bench_tools import prefill_flops
    _register()
    config = {"kinds": ["toy", "attention_bias", "toy"], "schedule": [0, 1, 2, 1], "architectures": ["ToyForTests"]}
    (tmp_path / "config.json").write_text(json.dumps(config))
    assert cli.main(["plan", "--model", str(tmp_path), "--dtype", "float32", "--context", "128", "--sessions", "2"]) == 0
    out = capsys.readouterr().out
    attention = (HEADS * HD + 2 * KV * HD) * (HIDDEN + 1) + HIDDEN * HEADS * HD
    ffn = 3 * INNER * HIDDEN
    layers = 2 * (HIDDEN * HIDDEN + ffn + 2 * HIDDEN) + attention + ffn + 2 * HIDDEN
    weights = 4 * (2 * VOCAB * HIDDEN + HIDDEN + layers)
    assert f"kv       : {2 * KV * HD * 4} bytes per token; 2 x 128 tokens" in out      # one attention layer keeps pages
    step = 4 * (VOCAB * HIDDEN + HIDDEN + layers + attention + ffn + 2 * HIDDEN)       # layer 1 is visited twice
    assert f"decode   : {step / 2**20:.1f} MiB read per token" in out
    engine, _ = _engine_and_weights(config, "float32")
    assert engine.model.weight_bytes() == weights and engine.model.step_param_bytes() == step
    assert engine.describe()["layer_kinds"] == "2 x toy_running_mean+swiglu, 1 x gqa_attention+swiglu"
    T = 10
    pairs = T * (T + 1) / 2
    per_attention = 2 * T * (2 * HEADS * HD + 2 * KV * HD) * HIDDEN + 4 * HEADS * HD * pairs
    want = 2 * (2 * T * HIDDEN * HIDDEN) + 2 * per_attention + 4 * (2 * T * ffn) + 2 * VOCAB * HIDDEN
    assert prefill_flops(engine, T) == want
