"""Weights: the safetensors reader and writer, the by-name binder's one error, the random
model (CPU)."""
import json
import os
import struct

import pytest
import torch

import helpers
import mini_llama_cpp_release_b200 as ml
from mini_llama_cpp_release_b200.config import ModelConfig, build_model_spec
from mini_llama_cpp_release_b200.engine.model import build_parts
from mini_llama_cpp_release_b200.weights import (Checkpoint, SafetensorsError, SafetensorsFile, WeightError, compare,
                                                 expected_tensors, save_safetensors)
from mini_llama_cpp_release_b200.weights.loader import device_dtype


def test_writer_and_reader_agree_with_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3)}
    ours = str(tmp_path / "ours.safetensors")
    save_safetensors(ours, tensors, metadata={"k": "v"})
    theirs = load_file(ours)
    for k in tensors:
        assert torch.equal(theirs[k], tensors[k])
    other = str(tmp_path / "theirs.safetensors")
    save_file(tensors, other)
    with SafetensorsFile(other) as f:
        for k in tensors:
            assert torch.equal(f.read(k), tensors[k]) and f.entries[k].shape == tuple(tensors[k].shape)


def _write_raw(path, header: dict, data: bytes):
    blob = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)) + blob + data)


def test_broken_files_are_refused_with_the_reason(tmp_path):
    p = str(tmp_path / "x.safetensors")
    _write_raw(p, {"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="outside the file"):
        SafetensorsFile(p)
    _write_raw(p, {"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}, b"\0" * 12)
    with pytest.raises(SafetensorsError, match="needs 16"):
        SafetensorsFile(p)
    _write_raw(p, {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                   "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12)
    with pytest.raises(SafetensorsError, match="overlap"):
        SafetensorsFile(p)
    _write_raw(p, {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 12)
    with pytest.raises(SafetensorsError, match="trailing"):
        SafetensorsFile(p)
    _write_raw(p, {"a": {"dtype": "Q4_0", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(p)
    with open(p, "wb") as f:
        f.write(b"\x05")
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        Checkpoint(str(tmp_path / "empty"))


def _specs(name):
    spec = build_model_spec(ModelConfig.from_dict(helpers.CONFIGS[name]))
    return expected_tensors(build_parts(spec).all_parts())


def test_expected_tensors_carry_the_checkpoints_names_and_shapes():
    specs = _specs("B")
    assert specs["model.embed_tokens.weight"].shape == (1000, 128)
    assert specs["model.layers.2.self_attn.k_proj.weight"].shape == (16, 128)
    assert specs["model.layers.0.self_attn.q_proj.bias"].shape == (128,)
    assert specs["model.layers.1.mlp.down_proj.weight"].shape == (128, 344)
    assert specs["lm_head.weight"].shape == (1000, 128) and specs["lm_head.weight"].stored
    tied = _specs("A")
    assert "lm_head.weight" not in tied and len(tied) == 2 + 2 * 12


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = helpers.model_folder("A")
    from safetensors.torch import load_file
    w = load_file(os.path.join(folder, "model.safetensors"))
    del w["model.layers.1.self_attn.q_proj.bias"]
    del w["model.norm.weight"]
    w["model.layers.0.mlp.up_proj.weight"] = torch.zeros(176, 63)
    w["model.layers.7.surprise"] = torch.zeros(2)
    bad = tmp_path / "bad"
    bad.mkdir()
    save_safetensors(str(bad / "model.safetensors"), w)
    ModelConfig.from_dict(helpers.TINY_A).save(str(bad))
    with Checkpoint(str(bad)) as ck:
        lines = "\n".join(compare(ck.entries, _specs("A")))
    assert "missing tensors (2)" in lines and "model.norm.weight" in lines and "q_proj.bias" in lines
    assert "unexpected tensors (1)" in lines and "model.layers.7.surprise" in lines
    assert "wrong shapes (1)" in lines and "[176, 63]" in lines and "[176, 64]" in lines


def test_tied_head_in_the_file_is_tolerated_only_when_tied():
    specs = _specs("A")
    from mini_llama_cpp_release_b200.weights.safetensors_io import TensorEntry
    entries = {n: TensorEntry(n, "BF16", tuple(s.shape), 0, 0, "f") for n, s in specs.items()}
    entries["lm_head.weight"] = TensorEntry("lm_head.weight", "BF16", (512, 64), 0, 0, "f")
    assert compare(entries, specs, ignore_extra=["lm_head.weight"]) == []
    assert "unexpected" in compare(entries, specs)[0]
    entries["model.layers.0.self_attn.rotary_emb.inv_freq"] = TensorEntry("x", "F32", (8,), 0, 0, "f")
    assert compare(entries, specs, ignore_extra=["lm_head.weight"]) == []


def test_element_types_on_the_device():
    bf, f32 = torch.bfloat16, torch.float32
    assert device_dtype("BF16", "matrix", bf) == bf and device_dtype("F16", "matrix", bf) == bf
    assert device_dtype("F32", "matrix", bf) == f32          # stored in 32-bit stays 32-bit
    assert device_dtype("BF16", "matrix", f32) == f32
    assert device_dtype("I64", "int_table", bf) == torch.int32


def test_random_model_is_a_function_of_config_and_seed(tmp_path):
    cfg = ModelConfig.from_dict(helpers.TINY_A)
    a = ml.write_random_model(cfg, str(tmp_path / "a"), 5)
    b = ml.write_random_model(cfg, str(tmp_path / "b"), 5)
    c = ml.write_random_model(cfg, str(tmp_path / "c"), 6)
    ra, rb, rc = (open(os.path.join(f, "model.safetensors"), "rb").read() for f in (a, b, c))
    assert ra == rb and ra != rc
    with Checkpoint(a) as ck:
        assert compare(ck.entries, _specs("A")) == []
        gain = ck.read("model.layers.0.input_layernorm.weight").float()
        bias = ck.read("model.layers.0.self_attn.k_proj.bias").float()
        mat = ck.read("model.embed_tokens.weight").float()
        assert ck.entries["model.embed_tokens.weight"].dtype == "BF16"
    assert abs(float(gain.mean()) - 1.0) < 0.02 and 0.005 < float(gain.std()) < 0.04
    assert abs(float(bias.mean())) < 0.02 and float(bias.abs().max()) > 0
    assert 0.015 < float(mat.std()) < 0.025
    assert ModelConfig.from_folder(a) == cfg
