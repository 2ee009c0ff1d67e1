"""Safetensors reading, binding by name, the one error that lists everything, random weights (no GPU)."""
import json
import os

import pytest
import torch

from aegean_tge_b200 import WeightError, architecture_of, write_random_model
from aegean_tge_b200.parts.base import BuildEnv
from aegean_tge_b200.models.decoder import DecoderModel
from aegean_tge_b200.weights import ModelFiles, WeightFileError, check_against_manifest, write_safetensors
from aegean_tge_b200.weights.loader import device_dtype
from conftest import TINY_A, TINY_B


def _model(raw, dtype=torch.float32):
    arch = architecture_of(raw)
    spec = arch.build_spec(arch.parse_config(raw))
    env = BuildEnv(dtype=dtype, device=torch.device("cpu"), hidden_size=spec.hidden_size, max_positions=32,
                   page_size=16, ops=None)
    return DecoderModel(spec, env)


def test_round_trip_of_every_dtype(tmp_path):
    tensors = {"f": torch.randn(3, 5), "b": torch.randn(4, 2).to(torch.bfloat16), "i": torch.arange(6, dtype=torch.int32),
               "l": torch.arange(4, dtype=torch.int64), "s": torch.tensor(2.5)}
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, tensors)
    files = ModelFiles(str(tmp_path))
    assert set(files.names()) == set(tensors)
    for name, tensor in tensors.items():
        got = files.read(name)
        assert got.dtype == tensor.dtype and torch.equal(got, tensor)
    # the independent reader agrees
    from safetensors import safe_open
    with safe_open(path, framework="pt") as handle:
        assert torch.equal(handle.get_tensor("b"), tensors["b"])


def test_random_model_folder_is_seeded_and_complete(tmp_path):
    a, b, c = str(tmp_path / "a"), str(tmp_path / "b"), str(tmp_path / "c")
    write_random_model(a, TINY_A, seed=0)
    write_random_model(b, TINY_A, seed=0)
    write_random_model(c, TINY_A, seed=1)
    fa, fb, fc = ModelFiles(a), ModelFiles(b), ModelFiles(c)
    assert json.load(open(os.path.join(a, "config.json")))["hidden_size"] == 64
    manifest = _model(TINY_A).manifest()
    assert set(fa.names()) == set(manifest)                       # tied: no lm_head.weight
    assert "lm_head.weight" not in manifest
    for name in fa.names():
        assert torch.equal(fa.read(name), fb.read(name))
    assert not torch.equal(fa.read("model.embed_tokens.weight"), fc.read("model.embed_tokens.weight"))
    w = fa.read("model.layers.0.mlp.down_proj.weight")
    assert w.shape == (64, 176) and abs(float(w.std()) - 0.02) < 0.002
    n = fa.read("model.norm.weight")
    assert float(n.min()) >= 0.9 and float(n.max()) <= 1.1 and n.dtype == torch.float32
    write_random_model(str(tmp_path / "d"), TINY_B, seed=1, dtype="bfloat16")
    fd = ModelFiles(str(tmp_path / "d"))
    assert fd.read("lm_head.weight").dtype == torch.bfloat16
    assert fd.read("model.layers.2.self_attn.q_proj.bias").dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = str(tmp_path / "m")
    write_random_model(folder, TINY_B, seed=3)
    files = ModelFiles(folder)
    tensors = {name: files.read(name).clone() for name in files.names()}
    del tensors["model.layers.1.self_attn.k_proj.bias"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.mlp.up_proj.weight"] = torch.zeros(255, 96)
    tensors["model.layers.7.extra.weight"] = torch.zeros(2)
    tensors["model.norm.weight"] = torch.ones(96, dtype=torch.int32)
    model = _model(TINY_B)
    with pytest.raises(WeightError) as error:
        check_against_manifest({n: (t.dtype, tuple(t.shape)) for n, t in tensors.items()}, model.manifest())
    e = error.value
    assert e.missing == ["lm_head.weight", "model.layers.1.self_attn.k_proj.bias"]
    assert e.unexpected == ["model.layers.7.extra.weight"]
    assert len(e.mismatched) == 2
    text = str(e)
    assert "[255, 96]" in text and "[256, 96]" in text and "model.norm.weight" in text
    assert "lm_head.weight" in text and "model.layers.7.extra.weight" in text


def test_load_checkpoint_raises_the_same_error(tmp_path):
    from aegean_tge_b200.weights import load_checkpoint
    folder = str(tmp_path / "m")
    write_random_model(folder, TINY_A, seed=3)
    files = ModelFiles(folder)
    tensors = {name: files.read(name).clone() for name in files.names() if "post_attention" not in name}
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    model = _model(TINY_A)
    with pytest.raises(WeightError) as error:
        load_checkpoint(model, folder)
    assert len(error.value.missing) == 2


def test_dtype_by_role():
    from aegean_tge_b200.parts.base import ParamSpec
    assert device_dtype(ParamSpec((2, 2), "matrix"), torch.bfloat16) == torch.bfloat16
    assert device_dtype(ParamSpec((2, 2), "matrix"), torch.float32) == torch.float32
    assert device_dtype(ParamSpec((2,), "vector"), torch.bfloat16) == torch.float32     # 32-bit stays 32-bit
    assert device_dtype(ParamSpec((2,), "table"), torch.bfloat16) == torch.int32


def test_loaded_model_fuses_and_interleaves(tmp_path):
    """q/k/v rows are concatenated, gate/up rows interleaved, the tied head is the embedding itself."""
    from aegean_tge_b200.weights import load_checkpoint
    folder = str(tmp_path / "m")
    write_random_model(folder, TINY_A, seed=5)
    files = ModelFiles(folder)
    model = _model(TINY_A, torch.bfloat16)
    load_checkpoint(model, folder)
    mixer = model.blocks[1].mixer
    assert mixer.w_qkv.shape == (64 + 32 + 32, 64) and mixer.w_qkv.dtype == torch.bfloat16
    assert torch.equal(mixer.w_qkv[64:96], files.read("model.layers.1.self_attn.k_proj.weight").to(torch.bfloat16))
    assert mixer.b_qkv.dtype == torch.float32 and mixer.b_qkv.shape == (128,)
    ffn = model.blocks[0].feed_forward
    assert torch.equal(ffn.w_gate_up[0::2], files.read("model.layers.0.mlp.gate_proj.weight").to(torch.bfloat16))
    assert torch.equal(ffn.w_gate_up[1::2], files.read("model.layers.0.mlp.up_proj.weight").to(torch.bfloat16))
    assert model.head.weight.data_ptr() == model.embedding.weight.data_ptr()
    assert model.final_norm.weight.dtype == torch.float32


def test_bad_files_are_refused(tmp_path):
    with pytest.raises(WeightFileError):
        ModelFiles(str(tmp_path))
    (tmp_path / "model.safetensors").write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00{not json......}")
    with pytest.raises(WeightFileError):
        ModelFiles(str(tmp_path))
    (tmp_path / "model.safetensors").write_bytes(b"\xff\xff\xff\xff\xff\xff\xff\x7f")
    with pytest.raises(WeightFileError):
        ModelFiles(str(tmp_path))
