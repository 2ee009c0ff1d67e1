"""Each part of a layer alone, built from a PartSpec, against the plain functions."""
import math

import pytest
import torch

from helpers import TOL, batch_index, paged_cache, rel_error
from plain import ops_plain
from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]


def _env(dtype, hidden, max_positions=128):
    from aegean_tge_b200 import ops
    from aegean_tge_b200.parts.base import BuildEnv
    ops.core()
    return BuildEnv(dtype=dtype, device=DEV, hidden_size=hidden, max_positions=max_positions, page_size=16, ops=ops)


def _ctx(q_lens, starts, table):
    from aegean_tge_b200.parts.base import StepContext
    positions, seq_of_token, q_start, start_pos = batch_index(q_lens, starts, DEV)
    n = len(q_lens)
    return StepContext(num_tokens=sum(q_lens), num_seqs=n, token_ids=positions, positions=positions,
                       seq_of_token=seq_of_token, q_start=q_start, start_pos=start_pos,
                       ctx_len=torch.tensor([s + q for s, q in zip(starts, q_lens)], dtype=torch.int32, device=DEV),
                       slots=torch.arange(n, dtype=torch.int32, device=DEV), block_tables=[table],
                       max_q_len=max(q_lens), max_ctx_len=max(s + q for s, q in zip(starts, q_lens)),
                       host_q_lens=list(q_lens), host_start_pos=list(starts), host_slots=list(range(n)))


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from aegean_tge_b200.config import PartSpec
    from aegean_tge_b200.parts import NORMS, build_part
    part = build_part(NORMS, PartSpec("rmsnorm", {"size": 200, "eps": 3e-5}, {"weight": "w"}), _env(dtype, 200))
    assert part.param_specs()["weight"].shape == (200,) and part.param_specs()["weight"].role == "vector"
    gen = torch.Generator().manual_seed(0)
    w = 1 + 0.1 * torch.randn(200, generator=gen)
    x = torch.randn(9, 200, generator=gen) * 4
    part.load({"weight": w.to(DEV)})
    assert rel_error(part.forward(x.to(DEV)), plain.rms_norm(x.double(), w.double(), 3e-5)) < TOL[dtype]
    rows = torch.tensor([8, 2], dtype=torch.int32, device=DEV)
    assert rel_error(part.forward(x.to(DEV), rows=rows), plain.rms_norm(x[[8, 2]].double(), w.double(), 3e-5)) < TOL[dtype]
    assert part.fusable()[1] == 3e-5


def test_rope_part_tables_and_parameters():
    from aegean_tge_b200.config import PartSpec
    from aegean_tge_b200.parts import POSITIONS, build_part
    env = _env(torch.float32, 64, max_positions=300)
    part = build_part(POSITIONS, PartSpec("rope_neox", {"head_dim": 48, "theta": 5e4}), env)
    cos, sin, rotary = part.rotary_tables()
    ref_cos, ref_sin = plain.rope_tables(5e4, 48, 300)
    assert rotary == 48 and torch.equal(cos.cpu(), ref_cos.float()) and torch.equal(sin.cpu(), ref_sin.float())
    partial = build_part(POSITIONS, PartSpec("rope_neox", {"head_dim": 48, "theta": 5e4, "rotary_dim": 16}), env)
    assert partial.rotary_tables()[0].shape == (300, 8)
    with pytest.raises(ValueError):
        build_part(POSITIONS, PartSpec("rope_neox", {"head_dim": 48, "theta": 5e4, "rotary_dim": 50}), env)
    assert build_part(POSITIONS, PartSpec("none"), env).rotary_tables() == (None, None, 0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(dtype):
    from aegean_tge_b200.config import PartSpec
    from aegean_tge_b200.parts import FEED_FORWARDS, build_part
    hidden, inner = 72, 200
    part = build_part(FEED_FORWARDS, PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": inner},
                                              {"gate.weight": "g", "up.weight": "u", "down.weight": "d"}), _env(dtype, hidden))
    gen = torch.Generator().manual_seed(1)
    g, u, d = (torch.randn(s, generator=gen).to(dtype) * 0.2 for s in ((inner, hidden), (inner, hidden), (hidden, inner)))
    part.load({"gate.weight": g.to(DEV), "up.weight": u.to(DEV), "down.weight": d.to(DEV)})
    h = torch.randn(11, hidden, generator=gen).to(dtype)
    ref = plain.swiglu(h.double(), g.double(), u.double(), d.double())
    assert rel_error(part.forward(h.to(DEV), None), ref) < 2 * TOL[dtype]
    x = torch.randn(11, hidden, generator=gen)
    dx = x.to(DEV)
    assert part.forward_add(h.to(DEV), dx, None) is None
    assert rel_error(dx, x.double() + ref) < 2 * TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 20])
def test_attention_part_with_its_cache(dtype, window):
    """The mixer alone: products with bias, rotation, cache store, attention over old and new pages, output product."""
    from aegean_tge_b200.config import PartSpec
    from aegean_tge_b200.parts import MIXERS, LayerCache, build_part
    hidden, heads, kv, hd = 96, 6, 2, 16
    position = PartSpec("rope_neox", {"head_dim": hd, "theta": 1e4})
    spec = PartSpec("gqa_attention", {"hidden_size": hidden, "heads": heads, "kv_heads": kv, "head_dim": hd,
                                      "qkv_bias": True, "o_bias": False, "window": window, "position": position},
                    {f"{x}.{y}": f"{x}.{y}" for x in "qkvo" for y in ("weight", "bias")})
    part = build_part(MIXERS, spec, _env(dtype, hidden))
    assert part.cache_spec().window == window and part.state_spec() is None
    gen = torch.Generator().manual_seed(2)
    mk = lambda *s: (torch.randn(s, generator=gen) * 0.15).to(dtype)
    w = {"q.weight": mk(heads * hd, hidden), "k.weight": mk(kv * hd, hidden), "v.weight": mk(kv * hd, hidden),
         "o.weight": mk(hidden, heads * hd), "q.bias": mk(heads * hd).float(), "k.bias": mk(kv * hd).float(),
         "v.bias": mk(kv * hd).float()}
    part.load({k: v.to(DEV) for k, v in w.items()})
    # two requests: one continues after 21 cached positions, one starts
    q_lens, starts = [7, 5], [21, 0]
    total = [s + q for s, q in zip(starts, q_lens)]
    h_all = [torch.randn(n, hidden, generator=gen).to(dtype) for n in total]     # normed inputs of every position
    cos, sin = plain.rope_tables(1e4, hd, 64)
    def qkv_of(h):
        h = h.double()
        q = plain.apply_rope((h @ w["q.weight"].double().T + w["q.bias"].double()).view(-1, heads, hd), cos[:len(h)], sin[:len(h)])
        k = plain.apply_rope((h @ w["k.weight"].double().T + w["k.bias"].double()).view(-1, kv, hd), cos[:len(h)], sin[:len(h)])
        v = (h @ w["v.weight"].double().T + w["v.bias"].double()).view(-1, kv, hd)
        return q, k, v
    k_pages, v_pages, table, _, _ = paged_cache(total, kv, hd, 16, dtype, DEV, seed=3)
    refs = []
    for s, h in enumerate(h_all):
        q, k, v = qkv_of(h)
        for pos in range(starts[s]):                       # what earlier steps left in the cache
            page = int(table[s, pos // 16])
            k_pages[page, :, pos % 16] = k[pos].to(dtype)
            v_pages[page, :, pos % 16] = v[pos].to(dtype)
        a = plain.attention(q, k, v, window=window or 0).reshape(len(h), heads * hd)
        refs.append((a @ w["o.weight"].double().T)[starts[s]:])
    cache = LayerCache(paged={"k": k_pages, "v": v_pages}, group=0)
    ctx = _ctx(q_lens, starts, table)
    h_step = torch.cat([h[starts[s]:] for s, h in enumerate(h_all)]).to(DEV)
    out = part.forward(h_step, ctx, cache)
    assert rel_error(out, torch.cat(refs)) < 3 * TOL[dtype]
    x = torch.zeros(sum(q_lens), hidden, device=DEV)
    part.forward_add(h_step, x, ctx, cache)
    assert rel_error(x, torch.cat(refs)) < 3 * TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    from aegean_tge_b200.config import PartSpec
    from aegean_tge_b200.parts import EMBEDDINGS, HEADS, build_part
    env = _env(dtype, 40)
    sizes = {"vocab_size": 97, "hidden_size": 40}
    emb = build_part(EMBEDDINGS, PartSpec("token_embedding", sizes, {"weight": "e"}), env)
    head = build_part(HEADS, PartSpec("linear_head", sizes, {"weight": "e"}), env)
    table = (torch.randn(97, 40, generator=torch.Generator().manual_seed(4)) * 0.3).to(dtype)
    emb.load({"weight": table.to(DEV)}); head.load({"weight": table.to(DEV)})
    ids = torch.tensor([5, 96, 0, 5], dtype=torch.int32, device=DEV)
    x = emb.forward(ids)
    assert x.dtype == torch.float32 and torch.equal(x.cpu(), table[[5, 96, 0, 5]].float())
    logits = head.forward(x.to(dtype))
    assert logits.dtype == torch.float32 and rel_error(logits, table[[5, 96, 0, 5]].double() @ table.double().T) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_pre_norm_block_order(dtype):
    """x += mixer(norm1(x)); x += ffn(norm2(x)), with stand-in mixer and feed-forward that show the order."""
    from aegean_tge_b200.config import PartSpec
    from aegean_tge_b200.parts import BLOCKS, NORMS, FeedForward, LayerCache, Mixer, build_part
    env = _env(dtype, 64)

    class Doubler(Mixer):
        def forward(self, h, ctx, cache):
            return (h.float() * 2).to(h.dtype)

    class PlusOne(FeedForward):
        def forward(self, h, ctx):
            return (h.float() + 1).to(h.dtype)

    gen = torch.Generator().manual_seed(5)
    w1, w2 = 1 + 0.1 * torch.randn(64, generator=gen), 1 + 0.1 * torch.randn(64, generator=gen)
    n1 = build_part(NORMS, PartSpec("rmsnorm", {"size": 64, "eps": 1e-6}, {"weight": "a"}), env)
    n2 = build_part(NORMS, PartSpec("rmsnorm", {"size": 64, "eps": 1e-6}, {"weight": "b"}), env)
    n1.load({"weight": w1.to(DEV)}); n2.load({"weight": w2.to(DEV)})
    block = BLOCKS.get("pre_norm")(Doubler(PartSpec("x"), env), PlusOne(PartSpec("y"), env), n1, n2, env)
    x = torch.randn(6, 64, generator=gen)
    dx = x.to(DEV)
    assert block.forward(dx, None, LayerCache()) is None
    mid = x.double() + 2 * plain.rms_norm(x.double(), w1.double(), 1e-6)
    ref = mid + plain.rms_norm(mid, w2.double(), 1e-6) + 1
    assert rel_error(dx, ref) < 3 * TOL[dtype]
