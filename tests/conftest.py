"""Shared fixtures: two tiny configurations that differ in every size and option, and model folders
with seeded random weights made in temporary folders."""
import json
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

# tiny A: 2 layers, hidden 64, 4 query heads on 2 kv heads of 16, tied head
TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 176, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 256, "use_sliding_window": False,
    "hidden_act": "silu",
}
# tiny B: 3 layers, hidden 96, 3 query heads on 1 kv head of 32, separate head
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "intermediate_size": 256, "vocab_size": 384, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 512, "use_sliding_window": False,
    "hidden_act": "silu",
}
# tiny C: sizes that are no power of two anywhere, head_dim 48, 6 query heads on 2 kv heads, vocab 331
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 120, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 48, "intermediate_size": 200, "vocab_size": 331, "rope_theta": 50000.0, "rms_norm_eps": 3e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 384, "use_sliding_window": False,
    "hidden_act": "silu",
}
# tiny D: head_dim 64 (the TMA-fed attention kernels), 8 query heads on 2 kv heads, long positions
TINY_D = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 192, "num_attention_heads": 8, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 320, "vocab_size": 500, "rope_theta": 100000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 4096, "use_sliding_window": False,
    "hidden_act": "silu",
}
# tiny E: nothing is a multiple of 8 or 16 (head size 20, width 100, inner width 70, a prime vocabulary, as many
# kv heads as query heads, tied head): what the tensor-core and 16-byte kernels refuse goes to the plain ones
TINY_E = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 100, "num_attention_heads": 5, "num_key_value_heads": 5,
    "head_dim": 20, "intermediate_size": 70, "vocab_size": 97, "rope_theta": 2000.0, "rms_norm_eps": 2e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 300, "use_sliding_window": False,
    "hidden_act": "silu",
}
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2), "D": (TINY_D, 3), "E": (TINY_E, 4)}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """name -> folder with config.json and model.safetensors (float32 weights, seeded)."""
    from aegean_tge_b200 import write_random_model
    out = {}
    for name, (config, seed) in TINY.items():
        folder = tmp_path_factory.mktemp(f"tiny_{name}")
        write_random_model(str(folder), config, seed=seed, dtype="float32")
        out[name] = str(folder)
    return out
