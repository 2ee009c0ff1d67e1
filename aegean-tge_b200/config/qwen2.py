"""Typed configuration of the Qwen2.5 dense decoder, read from config.json.

Field-for-field this is what the reference takes from ``qwen2.*`` GGUF
metadata in ``read_config`` (src/models/qwen2.cpp:222-389) and keeps in
``Qwen2Config`` (include/tge/models/qwen2.hpp:42-94), under the names a
Hugging Face ``config.json`` gives them:

=========================== =====================================
reference key                config.json key
=========================== =====================================
block_count                  num_hidden_layers
embedding_length             hidden_size
feed_forward_length          intermediate_size
attention.head_count         num_attention_heads
attention.head_count_kv      num_key_value_heads (default: heads)
attention.key_length         head_dim (default: hidden / heads)
context_length               max_position_embeddings
layer_norm_rms_epsilon       rms_norm_eps (default 1e-6)
rope.freq_base               rope_theta (default 10000)
(output.weight present?)     tie_word_embeddings
eos / eos_token_ids          eos_token_id (int or list)
=========================== =====================================

No size or constant that config.json gives is repeated anywhere else in the
package.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, Dict, Tuple

from .common import ConfigError, read_config_json  # noqa: F401  (ConfigError is raised below)

ARCHITECTURE = "Qwen2ForCausalLM"


def _need_int(raw: Dict[str, Any], key: str, *, minimum: int = 1) -> int:
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: missing key '{key}'")
    value = raw[key]
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError(f"config.json: '{key}' must be >= {minimum}, got {value}")
    return value


def _opt_number(raw: Dict[str, Any], key: str, default: float) -> float:
    value = raw.get(key, default)
    if value is None:
        return default
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json: '{key}' must be a number, got {value!r}")
    if not math.isfinite(float(value)):
        raise ConfigError(f"config.json: '{key}' must be finite, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class Qwen2Config:
    num_hidden_layers: int
    hidden_size: int
    intermediate_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    vocab_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    end_token_ids: Tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)

    # -- derived sizes ----------------------------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        """Same quantity as the reference's ``kv_dim()`` (qwen2.hpp:81)."""
        return self.num_key_value_heads * self.head_dim

    def is_end_token(self, token: int) -> bool:
        """Mirrors ``Qwen2Config::is_end_token`` (qwen2.hpp:83-93)."""
        return token >= 0 and token in self.end_token_ids

    # -- construction -----------------------------------------------------
    @staticmethod
    def from_dict(raw: Dict[str, Any]) -> "Qwen2Config":
        layers = _need_int(raw, "num_hidden_layers")
        hidden = _need_int(raw, "hidden_size")
        inter = _need_int(raw, "intermediate_size")
        heads = _need_int(raw, "num_attention_heads")
        kv_heads = raw.get("num_key_value_heads")
        kv_heads = heads if kv_heads is None else _need_int(raw, "num_key_value_heads")
        if raw.get("head_dim") is None:
            # The reference defaults key_length to embedding_length / head_count
            # and refuses a remainder (qwen2.cpp:342-359).
            if hidden % heads != 0:
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not a multiple of "
                    f"num_attention_heads {heads} and no head_dim is given")
            head_dim = hidden // heads
        else:
            head_dim = _need_int(raw, "head_dim")
        max_pos = _need_int(raw, "max_position_embeddings")
        vocab = _need_int(raw, "vocab_size")
        if vocab >= 2 ** 31:
            raise ConfigError(f"config.json: vocab_size {vocab} does not fit 32-bit token ids")
        if heads % kv_heads != 0:
            # qwen2.cpp:352-355
            raise ConfigError(
                f"config.json: num_attention_heads {heads} is not a multiple of "
                f"num_key_value_heads {kv_heads}")
        if head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim {head_dim} must be even for rotary pairs")
        eps = _opt_number(raw, "rms_norm_eps", 1e-6)
        if not eps > 0.0:
            raise ConfigError(f"config.json: rms_norm_eps must be positive, got {eps}")
        theta = _opt_number(raw, "rope_theta", 10000.0)
        if not theta > 0.0:
            raise ConfigError(f"config.json: rope_theta must be positive, got {theta}")
        # The reference never windows attention (the causal mask is the loop
        # bound, qwen2.cpp:1276) and rejects rope scaling kinds it does not
        # know (qwen2.cpp:274-279).  Neither exists in this architecture.
        if raw.get("use_sliding_window", False):
            raise ConfigError("config.json: use_sliding_window=true is not part of this architecture")
        scaling = raw.get("rope_scaling")
        if scaling not in (None, {}):
            raise ConfigError(f"config.json: rope_scaling {scaling!r} is not supported")
        partial = raw.get("partial_rotary_factor", 1.0)
        if partial not in (None, 1, 1.0):
            # qwen2.cpp:365-369 refuses a rotary width below the head size.
            raise ConfigError(f"config.json: partial_rotary_factor {partial!r} is not supported")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act must be 'silu', got {act!r}")
        tie = raw.get("tie_word_embeddings", False)
        if not isinstance(tie, bool):
            raise ConfigError(f"config.json: tie_word_embeddings must be true or false, got {tie!r}")
        ends = raw.get("eos_token_id")
        if ends is None:
            end_ids: Tuple[int, ...] = ()
        elif isinstance(ends, int) and not isinstance(ends, bool):
            end_ids = (ends,)
        elif isinstance(ends, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in ends):
            end_ids = tuple(ends)
        else:
            # qwen2.cpp:284-304: a stop id that is no integer is an error.
            raise ConfigError(f"config.json: eos_token_id must be an integer or a list of integers, got {ends!r}")
        for e in end_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"config.json: eos_token_id {e} is outside the vocabulary of {vocab}")
        known = {
            "num_hidden_layers", "hidden_size", "intermediate_size", "num_attention_heads",
            "num_key_value_heads", "head_dim", "max_position_embeddings", "vocab_size",
            "rms_norm_eps", "rope_theta", "tie_word_embeddings", "eos_token_id", "torch_dtype",
            "use_sliding_window", "rope_scaling", "partial_rotary_factor", "hidden_act",
        }
        return Qwen2Config(
            num_hidden_layers=layers, hidden_size=hidden, intermediate_size=inter,
            num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
            max_position_embeddings=max_pos, vocab_size=vocab, rms_norm_eps=eps,
            rope_theta=theta, tie_word_embeddings=tie, end_token_ids=end_ids,
            torch_dtype=str(raw.get("torch_dtype", "bfloat16")),
            extra={k: v for k, v in raw.items() if k not in known},
        )

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {
            "architectures": [ARCHITECTURE],
            "model_type": "qwen2",
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "use_sliding_window": False,
            "torch_dtype": self.torch_dtype,
        }
        if self.end_token_ids:
            out["eos_token_id"] = (self.end_token_ids[0] if len(self.end_token_ids) == 1
                                   else list(self.end_token_ids))
        return out
