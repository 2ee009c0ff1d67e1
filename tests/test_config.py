"""Configuration reading and the architecture registry (no GPU)."""
import copy

import pytest

from aegean_tge_b200 import ConfigError, Qwen2Config, architecture_of, registered_architectures
from aegean_tge_b200.config import ModelSpec
from conftest import TINY_A, TINY_B


def test_fields_come_from_config_json():
    c = Qwen2Config.from_dict(TINY_A)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (2, 64, 4, 2, 16)
    assert (c.intermediate_size, c.vocab_size, c.max_position_embeddings) == (176, 256, 256)
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0 and c.tie_word_embeddings is True
    assert c.q_dim == 64 and c.kv_dim == 32


def test_defaults_follow_the_reference():
    raw = {k: v for k, v in TINY_B.items() if k not in ("rms_norm_eps", "rope_theta", "tie_word_embeddings")}
    raw.pop("num_key_value_heads")
    c = Qwen2Config.from_dict(raw)
    assert c.head_dim == 32                      # hidden / heads
    assert c.num_key_value_heads == c.num_attention_heads
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0 and c.tie_word_embeddings is False


@pytest.mark.parametrize("change,needle", [
    ({"num_hidden_layers": None}, "num_hidden_layers"),
    ({"hidden_size": 0}, "hidden_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"use_sliding_window": True}, "use_sliding_window"),
    ({"rope_scaling": {"type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"rope_theta": -1.0}, "rope_theta"),
    ({"eos_token_id": "stop"}, "eos_token_id"),
    ({"eos_token_id": 999}, "outside the vocabulary"),
    ({"partial_rotary_factor": 0.5}, "partial_rotary_factor"),
    ({"vocab_size": 2 ** 31}, "vocab_size"),
    ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
])
def test_bad_values_are_named(change, needle):
    raw = copy.deepcopy(TINY_A)
    raw.update(change)
    if change.get("num_hidden_layers", 0) is None:
        del raw["num_hidden_layers"]
    with pytest.raises(ConfigError) as error:
        Qwen2Config.from_dict(raw)
    assert needle in str(error.value)


def test_hidden_not_divisible_needs_head_dim():
    raw = copy.deepcopy(TINY_A)
    raw.pop("head_dim")
    raw["hidden_size"] = 66
    with pytest.raises(ConfigError):
        Qwen2Config.from_dict(raw)
    raw["head_dim"] = 16
    assert Qwen2Config.from_dict(raw).q_dim == 64        # q width kept apart from the hidden size


def test_end_tokens():
    raw = copy.deepcopy(TINY_A)
    raw["eos_token_id"] = [3, 7]
    c = Qwen2Config.from_dict(raw)
    assert c.is_end_token(3) and c.is_end_token(7) and not c.is_end_token(4) and not c.is_end_token(-1)
    assert Qwen2Config.from_dict(c.to_dict()).end_token_ids == (3, 7)


def test_registry_picks_by_name_and_lists_names_on_miss():
    assert "Qwen2ForCausalLM" in registered_architectures()
    arch = architecture_of(TINY_A)
    spec = arch.build_spec(arch.parse_config(TINY_A))
    assert isinstance(spec, ModelSpec) and len(spec.layers) == 2 and spec.schedule == (0, 1)
    with pytest.raises(ConfigError) as error:
        architecture_of({"architectures": ["NoSuchModel"]})
    assert "Qwen2ForCausalLM" in str(error.value) and "NoSuchModel" in str(error.value)
    with pytest.raises(ConfigError):
        architecture_of({})


def test_spec_carries_every_constant_and_ties_the_head():
    arch = architecture_of(TINY_A)
    spec = arch.build_spec(arch.parse_config(TINY_A))
    mixer = spec.layers[1].mixer
    assert mixer.params["heads"] == 4 and mixer.params["kv_heads"] == 2 and mixer.params["head_dim"] == 16
    assert mixer.params["qkv_bias"] is True and mixer.params["o_bias"] is False
    assert mixer.params["position"].params["theta"] == 10000.0
    assert spec.layers[0].mixer_norm.params["eps"] == 1e-6
    assert spec.head.weights["weight"] == spec.embedding.weights["weight"]          # tied
    spec_b = architecture_of(TINY_B).build_spec(Qwen2Config.from_dict(TINY_B))
    assert spec_b.head.weights["weight"] == "lm_head.weight"
    assert spec_b.layers[0].ffn_norm.params["eps"] == 1e-5


def test_schedule_and_cache_sharing_are_validated():
    import dataclasses
    arch = architecture_of(TINY_B)
    spec = arch.build_spec(arch.parse_config(TINY_B))
    dataclasses.replace(spec, schedule=(0, 1, 1, 2)).validate()               # a layer may run twice
    with pytest.raises(ValueError):
        dataclasses.replace(spec, schedule=(0, 5)).validate()
    layers = list(spec.layers)
    layers[2] = dataclasses.replace(layers[2], cache_from=0)
    dataclasses.replace(spec, layers=tuple(layers)).validate()
    layers[0] = dataclasses.replace(layers[0], cache_from=2)
    with pytest.raises(ValueError):
        dataclasses.replace(spec, layers=tuple(layers)).validate()
