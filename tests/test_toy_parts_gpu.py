"""Toy parts defined here and stepped through the engine without touching the package: a feed-forward
with routing (top-2 of a few small experts, router in float32), a position encoding the fused
rotate-and-store kernel does not know (interleaved pairs, rotated over part of the head), and a norm
with a bias.  None of them is anyone's model; they show that a part is chosen by data, layer by layer,
and needs only the interface of its base class."""
import math
import random

import pytest
import torch

from helpers import MODEL_TOL, rel_error
from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

HIDDEN, VOCAB, HEADS, KV, HD, INNER = 40, 83, 4, 2, 16, 48
EXPERTS, EXPERT_INNER, TOP = 5, 24, 2
ROTATED, THETA = 12, 300.0            # interleaved pairs over the first 12 of 16 dims


def _register():
    from aegean_tge_b200.config.model_spec import LayerSpec, ModelSpec, PartSpec
    from aegean_tge_b200.parts.base import (FEED_FORWARDS, NORMS, POSITIONS, FeedForward, Norm, ParamSpec,
                                            PositionEncoding)
    from aegean_tge_b200.registry import Architecture, register_architecture, registered_architectures
    from aegean_tge_b200.weights import normal, uniform

    if "toy_routed" not in FEED_FORWARDS.names():
        @FEED_FORWARDS.register("toy_routed")
        class Routed(FeedForward):
            """out_t = sum over the top-2 experts e of softmax-over-the-two(router_t)[e] * W2_e gelu(W1_e h_t).

            Router logits in float32; experts visited in index order, so a token's sum has a fixed order
            whatever else is in the batch."""

            def __init__(self, spec, env):
                super().__init__(spec, env)
                p = spec.params
                self.hidden, self.experts, self.inner, self.top = (int(p[k]) for k in
                                                                   ("hidden_size", "experts", "inner", "top"))

            def param_specs(self):
                return {"router": ParamSpec((self.experts, self.hidden), role="vector"),
                        "w1": ParamSpec((self.experts, self.inner, self.hidden)),
                        "w2": ParamSpec((self.experts, self.hidden, self.inner))}

            def load(self, tensors):
                self.router, self.w1, self.w2 = tensors["router"], tensors["w1"], tensors["w2"]

            def forward(self, h, ctx):
                logits = h.float() @ self.router.float().T                       # [T, E] float32
                best, chosen = torch.topk(logits, self.top, dim=-1)
                gate = torch.softmax(best, dim=-1)
                out = torch.zeros(h.shape, dtype=torch.float32, device=h.device)
                for e in range(self.experts):                                    # fixed order per token
                    rows, which = torch.nonzero(chosen == e, as_tuple=True)
                    if rows.numel() == 0:
                        continue
                    inner = torch.nn.functional.gelu(h[rows].float() @ self.w1[e].float().T)
                    out[rows] += gate[rows, which][:, None] * (inner @ self.w2[e].float().T)
                return out.to(h.dtype)

    if "toy_rope_pairs" not in POSITIONS.names():
        @POSITIONS.register("toy_rope_pairs")
        class RopePairs(PositionEncoding):
            """Rotates the pairs (2i, 2i+1) of the first ``rotated`` dims; the rest passes through."""

            def __init__(self, spec, env):
                super().__init__(spec, env)
                self.rotated, self.theta = int(spec.params["rotated"]), float(spec.params["theta"])
                i = torch.arange(self.rotated // 2, dtype=torch.float32)
                self.freq = torch.pow(torch.tensor(self.theta), -2.0 * i / self.rotated).to(env.device)

            def param_specs(self):
                return {}

            def load(self, tensors):
                pass

            def apply(self, q, k, positions):
                angle = positions.float()[:, None] * self.freq[None, :]            # [T, rotated/2]
                c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
                for x in (q, k):
                    even, odd = x[..., 0:self.rotated:2].float().clone(), x[..., 1:self.rotated:2].float().clone()
                    x[..., 0:self.rotated:2] = (even * c - odd * s).to(x.dtype)
                    x[..., 1:self.rotated:2] = (even * s + odd * c).to(x.dtype)

    if "toy_layernorm" not in NORMS.names():
        @NORMS.register("toy_layernorm")
        class LayerNorm(Norm):
            """(x - mean) / sqrt(var + eps) * w + b over the float32 stream."""

            def __init__(self, spec, env):
                super().__init__(spec, env)
                self.size, self.eps = int(spec.params["size"]), float(spec.params["eps"])

            def param_specs(self):
                return {"weight": ParamSpec((self.size,), role="vector"), "bias": ParamSpec((self.size,), role="vector")}

            def load(self, tensors):
                self.weight, self.bias = tensors["weight"], tensors["bias"]

            def forward(self, x, rows=None):
                if rows is not None:
                    x = x[rows.long()]
                out = torch.nn.functional.layer_norm(x, (self.size,), self.weight, self.bias, self.eps)
                return out.to(self.env.dtype)

    def build_spec(config):
        position = PartSpec(config["position"], {"head_dim": HD, "theta": THETA, "rotated": ROTATED})
        def norm(name):
            if config["norm"] == "toy_layernorm":
                return PartSpec("toy_layernorm", {"size": HIDDEN, "eps": 1e-5}, {"weight": name + ".w", "bias": name + ".b"})
            return PartSpec("rmsnorm", {"size": HIDDEN, "eps": 1e-5}, {"weight": name + ".w"})
        layers = []
        for n, kind in enumerate(config["ffn"]):
            p = f"layers.{n}."
            mixer = PartSpec("gqa_attention",
                             {"hidden_size": HIDDEN, "heads": HEADS, "kv_heads": KV, "head_dim": HD, "qkv_bias": True,
                              "o_bias": False, "window": None, "position": position},
                             {f"{x}.{y}": p + f"{x}.{y}" for x in "qkvo" for y in ("weight", "bias")})
            if kind == "routed":
                ffn = PartSpec("toy_routed", {"hidden_size": HIDDEN, "experts": EXPERTS, "inner": EXPERT_INNER, "top": TOP},
                               {x: p + x for x in ("router", "w1", "w2")})
            else:
                ffn = PartSpec("swiglu", {"hidden_size": HIDDEN, "intermediate_size": INNER},
                               {f"{x}.weight": p + f"{x}.weight" for x in ("gate", "up", "down")})
            layers.append(LayerSpec("pre_norm", mixer, ffn, norm(p + "norm1"), norm(p + "norm2")))
        sizes = {"vocab_size": VOCAB, "hidden_size": HIDDEN}
        return ModelSpec("ToyPartsForTests", HIDDEN, VOCAB, 256, tuple(layers), tuple(range(len(layers))),
                         PartSpec("token_embedding", sizes, {"weight": "embed"}), norm("final_norm"),
                         PartSpec("linear_head", sizes, {"weight": "head"}))

    def random_plan(config):
        def mat(*shape, scale=0.1):
            return tuple(shape), "matrix", normal(scale)
        def vec(n, around=0.0):
            return (n,), "vector", (uniform(around - 0.08, around + 0.08) if around else normal(0.05))
        def norm(name):
            yield (name + ".w", *vec(HIDDEN, 1.0))
            if config["norm"] == "toy_layernorm":
                yield (name + ".b", *vec(HIDDEN))
        yield ("embed", *mat(VOCAB, HIDDEN))
        yield ("head", *mat(VOCAB, HIDDEN))
        yield from norm("final_norm")
        for n, kind in enumerate(config["ffn"]):
            p = f"layers.{n}."
            yield from norm(p + "norm1")
            yield from norm(p + "norm2")
            yield (p + "q.weight", *mat(HEADS * HD, HIDDEN))
            yield (p + "k.weight", *mat(KV * HD, HIDDEN))
            yield (p + "v.weight", *mat(KV * HD, HIDDEN))
            yield (p + "o.weight", *mat(HIDDEN, HEADS * HD))
            yield (p + "q.bias", *vec(HEADS * HD))
            yield (p + "k.bias", *vec(KV * HD))
            yield (p + "v.bias", *vec(KV * HD))
            if kind == "routed":
                # a router in float32 with well separated rows, so that bfloat16 rounding of h cannot flip a choice
                yield p + "router", (EXPERTS, HIDDEN), "vector", normal(2.0)
                yield (p + "w1", *mat(EXPERTS, EXPERT_INNER, HIDDEN))
                yield (p + "w2", *mat(EXPERTS, HIDDEN, EXPERT_INNER))
            else:
                for x, shape in (("gate", (INNER, HIDDEN)), ("up", (INNER, HIDDEN)), ("down", (HIDDEN, INNER))):
                    yield (p + f"{x}.weight", *mat(*shape))

    if "ToyPartsForTests" not in registered_architectures():
        register_architecture(Architecture("ToyPartsForTests", parse_config=lambda raw: raw, build_spec=build_spec,
                                           random_plan=random_plan))


# ---- the same toy architecture on whole sequences, float64, no cache --------------------------------
def _plain_norm(config, x, w, name):
    if config["norm"] == "toy_layernorm":
        mean = x.mean(-1, keepdim=True)
        var = ((x - mean) ** 2).mean(-1, keepdim=True)
        return (x - mean) / torch.sqrt(var + 1e-5) * w[name + ".w"] + w[name + ".b"]
    return plain.rms_norm(x, w[name + ".w"], 1e-5)


def _plain_position(config, x, T):
    """x [T, heads, HD] float64"""
    if config["position"] == "rope_neox":
        cos, sin = plain.rope_tables(THETA, HD, T)
        return plain.apply_rope(x, cos, sin)
    out = x.clone()
    for i in range(ROTATED // 2):
        freq = THETA ** (-2.0 * i / ROTATED)
        angle = torch.arange(T, dtype=torch.float64) * freq
        c, s = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
        out[..., 2 * i] = x[..., 2 * i] * c - x[..., 2 * i + 1] * s
        out[..., 2 * i + 1] = x[..., 2 * i] * s + x[..., 2 * i + 1] * c
    return out


def _plain_routed(h, w, p):
    out = torch.zeros_like(h)
    margins = []
    for t in range(h.shape[0]):
        logits = w[p + "router"] @ h[t]
        order = torch.argsort(logits, descending=True)
        margins.append(float(logits[order[TOP - 1]] - logits[order[TOP]]))
        top = order[:TOP]
        gate = torch.softmax(logits[top], dim=-1)
        for g, e in zip(gate, top):
            inner = w[p + "w1"][e] @ h[t]
            inner = 0.5 * inner * (1.0 + torch.erf(inner / math.sqrt(2.0)))
            out[t] += g * (w[p + "w2"][e] @ inner)
    return out, min(margins)


def _plain_logits(config, w, tokens):
    T = len(tokens)
    x = plain.embed(w["embed"], tokens)
    smallest_margin = float("inf")
    for n, kind in enumerate(config["ffn"]):
        p = f"layers.{n}."
        h = _plain_norm(config, x, w, p + "norm1")
        q = _plain_position(config, (h @ w[p + "q.weight"].T + w[p + "q.bias"]).view(T, HEADS, HD), T)
        k = _plain_position(config, (h @ w[p + "k.weight"].T + w[p + "k.bias"]).view(T, KV, HD), T)
        v = (h @ w[p + "v.weight"].T + w[p + "v.bias"]).view(T, KV, HD)
        x = x + plain.attention(q, k, v).reshape(T, HEADS * HD) @ w[p + "o.weight"].T
        h = _plain_norm(config, x, w, p + "norm2")
        if kind == "routed":
            y, margin = _plain_routed(h, w, p)
            smallest_margin = min(smallest_margin, margin)
            x = x + y
        else:
            x = x + plain.swiglu(h, w[p + "gate.weight"], w[p + "up.weight"], w[p + "down.weight"])
    return (_plain_norm(config, x, w, "final_norm") @ w["head"].T).float(), smallest_margin


def _engine_and_weights(config, dtype):
    from aegean_tge_b200 import Engine
    _register()
    engine = Engine(random_config=dict(config, architectures=["ToyPartsForTests"]), seed=11, dtype=dtype, context=256,
                    max_tokens=512, max_requests=4)
    model = engine.model
    w = {"embed": model.embedding.weight, "head": model.head.weight}
    def norm(name, part):
        w[name + ".w"] = part.weight
        if config["norm"] == "toy_layernorm":
            w[name + ".b"] = part.bias
    norm("final_norm", model.final_norm)
    for n, block in enumerate(model.blocks):
        p = f"layers.{n}."
        norm(p + "norm1", block.mixer_norm)
        norm(p + "norm2", block.ffn_norm)
        w[p + "q.weight"], w[p + "k.weight"], w[p + "v.weight"] = block.mixer.w_qkv.split([HEADS * HD, KV * HD, KV * HD])
        w[p + "q.bias"], w[p + "k.bias"], w[p + "v.bias"] = block.mixer.b_qkv.split([HEADS * HD, KV * HD, KV * HD])
        w[p + "o.weight"] = block.mixer.w_o
        if config["ffn"][n] == "routed":
            for x in ("router", "w1", "w2"):
                w[p + x] = getattr(block.feed_forward, x)
        else:
            gu = block.feed_forward.w_gate_up
            w[p + "gate.weight"], w[p + "up.weight"] = gu[0::2], gu[1::2]
            w[p + "down.weight"] = block.feed_forward.w_down
    return engine, {name: t.double().cpu() for name, t in w.items()}


CONFIGS = {
    "routed_between_dense": {"ffn": ["dense", "routed", "dense", "routed"], "position": "rope_neox", "norm": "rmsnorm"},
    "pairs_and_layernorm": {"ffn": ["dense", "dense"], "position": "toy_rope_pairs", "norm": "toy_layernorm"},
    "all_three": {"ffn": ["routed", "dense"], "position": "toy_rope_pairs", "norm": "toy_layernorm"},
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", list(CONFIGS))
def test_toy_feed_forward_position_and_norm(which, dtype):
    from aegean_tge_b200.engine import Portion
    config = CONFIGS[which]
    engine, w = _engine_and_weights(config, dtype)
    # Where two experts' router logits nearly tie, rounding may pick the other one, and such a row says
    # nothing about the engine: take the first draw of tokens whose smallest margin is clear.
    need, len_a, len_b = (0.35, 40, 17) if dtype == "bfloat16" else (1e-3, 70, 33)
    for seed in range(400):
        rnd = random.Random(seed)
        a = [rnd.randrange(VOCAB) for _ in range(len_a)]
        b = [rnd.randrange(VOCAB) for _ in range(len_b)]
        (ref_a, margin_a), (ref_b, margin_b) = _plain_logits(config, w, a), _plain_logits(config, w, b)
        if min(margin_a, margin_b) >= need:
            break
    else:
        raise AssertionError("no draw of tokens with clear router margins")
    full = lambda r, t: Portion(r, t, list(range(len(t))))
    c, d = (2 * len_a) // 5 + 1, len_b // 2 + 1
    got_a, got_b = [], []
    got_a.append(engine.runner.step([full("a", a[:c])]))
    out = engine.runner.step([full("a", a[c:c + 1]), full("b", b[:d])])
    got_a.append(out[:1]); got_b.append(out[1:])
    out = engine.runner.step([full("b", b[d:d + 2]), full("a", a[c + 1:len_a - 2])])
    got_b.append(out[:2]); got_a.append(out[2:])
    out = engine.runner.step([full("a", a[len_a - 2:]), full("b", b[d + 2:])])
    got_a.append(out[:2]); got_b.append(out[2:])
    got_a, got_b = torch.cat(got_a), torch.cat(got_b)
    assert rel_error(got_a, ref_a) < MODEL_TOL[dtype]
    assert rel_error(got_b, ref_b) < MODEL_TOL[dtype]
    engine.runner.finish("a"); engine.runner.finish("b")
    engine.cache.check()


def test_toy_parts_generate_through_the_entry_point():
    """The scheduler, the sampler and the cache serve the toy architecture as they serve any other."""
    _register()
    from aegean_tge_b200 import Engine
    config = dict(CONFIGS["all_three"], architectures=["ToyPartsForTests"])
    outputs = []
    for budget, pages in ((64, 64), (8, 12)):
        engine = Engine(random_config=config, seed=11, dtype="float32", context=128, num_pages=pages,
                        max_batch_tokens=budget, max_requests=3)
        outputs.append(engine.generate([[1, 2, 3, 4, 5, 6, 7, 8, 9], [10, 11], [12] * 20], n=12))
        engine.cache.check()
    assert outputs[0] == outputs[1]
    assert all(len(o) == 12 for o in outputs[0])
