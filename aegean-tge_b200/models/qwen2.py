"""The Qwen2.5 dense decoder as a ModelSpec, and its random weights.

Layer body in the reference's order (src/models/qwen2.cpp:2032-2123):
RMSNorm -> q/k/v projections with bias -> rotate-half RoPE on q and k ->
cache -> causal GQA -> output projection without bias -> residual ->
RMSNorm -> SwiGLU -> residual; after the last layer RMSNorm and the output
head, which is the embedding table when the model ties them.

Checkpoint tensor names are the Hugging Face ones, one-to-one with the
reference's GGUF names (src/models/qwen2.cpp:411-523):

==================================== ===============================
reference                             checkpoint
==================================== ===============================
token_embd.weight                     model.embed_tokens.weight
output_norm.weight                    model.norm.weight
output.weight                         lm_head.weight
blk.N.attn_norm.weight                model.layers.N.input_layernorm.weight
blk.N.attn_{q,k,v}.{weight,bias}      model.layers.N.self_attn.{q,k,v}_proj.{weight,bias}
blk.N.attn_output.weight              model.layers.N.self_attn.o_proj.weight
blk.N.ffn_norm.weight                 model.layers.N.post_attention_layernorm.weight
blk.N.ffn_{gate,up,down}.weight       model.layers.N.mlp.{gate,up,down}_proj.weight
==================================== ===============================

Both sides use rotate-half pairing, so no row permutation of q/k is needed.
"""
from __future__ import annotations

from typing import Dict, Iterator, Tuple

from ..config.model_spec import LayerSpec, ModelSpec, PartSpec
from ..config.qwen2 import ARCHITECTURE, Qwen2Config
from ..registry import Architecture, register_architecture
from ..weights.draws import Draw, normal, uniform


def build_spec(config: Qwen2Config) -> ModelSpec:
    hidden = config.hidden_size
    position = PartSpec("rope_neox", {"head_dim": config.head_dim, "theta": config.rope_theta})
    layers = []
    for n in range(config.num_hidden_layers):
        prefix = f"model.layers.{n}."
        mixer = PartSpec(
            "gqa_attention",
            {"hidden_size": hidden, "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
             "head_dim": config.head_dim, "qkv_bias": True, "o_bias": False, "window": None, "position": position},
            {"q.weight": prefix + "self_attn.q_proj.weight", "q.bias": prefix + "self_attn.q_proj.bias",
             "k.weight": prefix + "self_attn.k_proj.weight", "k.bias": prefix + "self_attn.k_proj.bias",
             "v.weight": prefix + "self_attn.v_proj.weight", "v.bias": prefix + "self_attn.v_proj.bias",
             "o.weight": prefix + "self_attn.o_proj.weight"})
        ffn = PartSpec(
            "swiglu", {"hidden_size": hidden, "intermediate_size": config.intermediate_size},
            {"gate.weight": prefix + "mlp.gate_proj.weight", "up.weight": prefix + "mlp.up_proj.weight",
             "down.weight": prefix + "mlp.down_proj.weight"})
        norm1 = PartSpec("rmsnorm", {"size": hidden, "eps": config.rms_norm_eps},
                         {"weight": prefix + "input_layernorm.weight"})
        norm2 = PartSpec("rmsnorm", {"size": hidden, "eps": config.rms_norm_eps},
                         {"weight": prefix + "post_attention_layernorm.weight"})
        layers.append(LayerSpec("pre_norm", mixer, ffn, norm1, norm2))
    sizes = {"vocab_size": config.vocab_size, "hidden_size": hidden}
    head_tensor = "model.embed_tokens.weight" if config.tie_word_embeddings else "lm_head.weight"
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=hidden, vocab_size=config.vocab_size,
        max_positions=config.max_position_embeddings, layers=tuple(layers),
        schedule=tuple(range(config.num_hidden_layers)),
        embedding=PartSpec("token_embedding", sizes, {"weight": "model.embed_tokens.weight"}),
        final_norm=PartSpec("rmsnorm", {"size": hidden, "eps": config.rms_norm_eps}, {"weight": "model.norm.weight"}),
        head=PartSpec("linear_head", sizes, {"weight": head_tensor}),
        end_token_ids=config.end_token_ids)


def tensor_shapes(config: Qwen2Config) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    """(name, shape, kind) of every checkpoint tensor; kind is matrix, bias or norm."""
    h, q, kv, ff = config.hidden_size, config.q_dim, config.kv_dim, config.intermediate_size
    yield "model.embed_tokens.weight", (config.vocab_size, h), "matrix"
    for n in range(config.num_hidden_layers):
        p = f"model.layers.{n}."
        yield p + "input_layernorm.weight", (h,), "norm"
        yield p + "self_attn.q_proj.weight", (q, h), "matrix"
        yield p + "self_attn.q_proj.bias", (q,), "bias"
        yield p + "self_attn.k_proj.weight", (kv, h), "matrix"
        yield p + "self_attn.k_proj.bias", (kv,), "bias"
        yield p + "self_attn.v_proj.weight", (kv, h), "matrix"
        yield p + "self_attn.v_proj.bias", (kv,), "bias"
        yield p + "self_attn.o_proj.weight", (h, q), "matrix"
        yield p + "post_attention_layernorm.weight", (h,), "norm"
        yield p + "mlp.gate_proj.weight", (ff, h), "matrix"
        yield p + "mlp.up_proj.weight", (ff, h), "matrix"
        yield p + "mlp.down_proj.weight", (h, ff), "matrix"
    yield "model.norm.weight", (h,), "norm"
    if not config.tie_word_embeddings:
        yield "lm_head.weight", (config.vocab_size, h), "matrix"


def random_plan(config: Qwen2Config) -> Iterator[Tuple[str, Tuple[int, ...], str, Draw]]:
    """Random weights: matrices and biases N(0, 0.02), norm weights 1 + U(-0.1, 0.1).

    (name, shape, role, draw) of every checkpoint tensor; matrices are stored in the run dtype, biases and
    norm weights in float32.
    """
    for name, shape, kind in tensor_shapes(config):
        if kind == "norm":
            yield name, shape, "vector", uniform(0.9, 1.1)
        else:
            yield name, shape, "matrix" if kind == "matrix" else "vector", normal(0.02)


register_architecture(Architecture(name=ARCHITECTURE, parse_config=Qwen2Config.from_dict, build_spec=build_spec,
                                   random_plan=random_plan))
