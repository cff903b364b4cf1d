"""Safetensors reading, the manifest check with its one error, random weights (no GPU).
The cases mirror test/model_param_validation_test.cpp of the reference."""
import json
import struct

import numpy as np
import pytest
import torch

import plain_model
import tiny_configs
from easy_gpt.cpp_b200.engine.model import Model
from easy_gpt.cpp_b200.registry import model_spec_from_config
from easy_gpt.cpp_b200.weights.loader import WeightError, load_checked
from easy_gpt.cpp_b200.weights.random_init import write_random_model
from easy_gpt.cpp_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors


def raw_file(path, header: dict, data: bytes = b"", header_len=None):
    hs = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(hs) if header_len is None else header_len) + hs + data)
    return path


def test_round_trip_keeps_stored_precision(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7), "c": torch.randn(2, 2).to(torch.float16),
         "ids": torch.arange(6, dtype=torch.int64).reshape(2, 3)}
    write_safetensors(tmp_path / "m.safetensors", t.items())
    with SafetensorsFile(tmp_path / "m.safetensors") as f:
        assert f.names() == ["a", "b", "c", "ids"]
        assert f.tensor("a").dtype == torch.bfloat16 and torch.equal(f.tensor("a"), t["a"])      # bfloat16 stays
        assert f.tensor("b").dtype == torch.float32 and torch.equal(f.tensor("b"), t["b"])       # 32-bit stays
        assert f.tensor("c").dtype == torch.float32 and torch.equal(f.tensor("c"), t["c"].float())
        assert f.tensor("ids").dtype == torch.int32 and f.tensor("ids").tolist() == [[0, 1, 2], [3, 4, 5]]
    # the plain reader sees the same numbers
    p = plain_model.read_safetensors(tmp_path / "m.safetensors")
    assert torch.equal(p["a"], t["a"].float()) and torch.equal(p["b"], t["b"])


@pytest.mark.parametrize("make, text", [
    (lambda p: p.write_bytes(b"\x01\x02"), "smaller than"),
    (lambda p: raw_file(p, {}, header_len=10_000), "exceeds the file size"),
    (lambda p: p.write_bytes(struct.pack("<Q", 4) + b"nope"), "not JSON"),
    (lambda p: raw_file(p, {"w": {"shape": [1], "data_offsets": [0, 4]}}, b"\0" * 4), "missing dtype"),
    (lambda p: raw_file(p, {"w": {"dtype": "I8", "shape": [4], "data_offsets": [0, 4]}}, b"\0" * 4), "Unsupported dtype"),
    (lambda p: raw_file(p, {"w": {"dtype": "F32", "shape": [], "data_offsets": [0, 4]}}, b"\0" * 4), "shape"),
    (lambda p: raw_file(p, {"w": {"dtype": "F32", "shape": [0], "data_offsets": [0, 0]}}), "bad dimension"),
    (lambda p: raw_file(p, {"w": {"dtype": "F32", "shape": [1], "data_offsets": [4, 0]}}, b"\0" * 4), "data_offsets"),
    (lambda p: raw_file(p, {"w": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 4), "past the end"),
    (lambda p: raw_file(p, {"w": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 4), "needs 8"),
])
def test_malformed_files_are_refused(tmp_path, make, text):
    path = tmp_path / "bad.safetensors"
    make(path)
    with pytest.raises(SafetensorsError, match=text):
        SafetensorsFile(path)


def test_missing_file():
    with pytest.raises(SafetensorsError, match="cannot open"):
        SafetensorsFile("/nonexistent/model.safetensors")


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = tiny_configs.write_tiny("B", tmp_path / "m")
    model = Model(model_spec_from_config(tiny_configs.CONFIG_B), "cpu", torch.float32)
    tensors = plain_model.read_safetensors(folder / "model.safetensors")
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["lm_head.weight"]                                   # untied: the head is required
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(64, 81)
    tensors["model.layers.2.self_attn.q_proj.bias"] = torch.zeros(191)
    tensors["model.layers.7.extra.weight"] = torch.zeros(2, 2)
    write_safetensors(folder / "broken.safetensors", tensors.items())
    with pytest.raises(WeightError) as e:
        load_checked(folder / "broken.safetensors", model.tensor_requests())
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "lm_head.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert [w[0] for w in err.wrong_shape] == ["model.layers.0.self_attn.k_proj.weight", "model.layers.2.self_attn.q_proj.bias"]
    text = str(err)
    assert "Missing required model weights: model.layers.1.mlp.up_proj.weight, lm_head.weight" in text
    assert "Unexpected tensors in the file: model.layers.7.extra.weight" in text
    assert "'model.layers.0.self_attn.k_proj.weight': expected [64, 80], got [64, 81]" in text


def test_tied_model_refuses_a_head_and_column_vectors_are_accepted(tmp_path):
    folder = tiny_configs.write_tiny("A", tmp_path / "m")
    model = Model(model_spec_from_config(tiny_configs.CONFIG_A), "cpu", torch.float32)
    tensors = plain_model.read_safetensors(folder / "model.safetensors")
    tensors["model.norm.weight"] = tensors["model.norm.weight"].reshape(-1, 1)      # [H, 1] like [H]
    write_safetensors(folder / "col.safetensors", tensors.items())
    got = load_checked(folder / "col.safetensors", model.tensor_requests())
    assert got["model.norm.weight"].shape == (64,)
    tensors["lm_head.weight"] = torch.zeros(256, 64)
    write_safetensors(folder / "head.safetensors", tensors.items())
    with pytest.raises(WeightError, match="Unexpected tensors in the file: lm_head.weight"):
        load_checked(folder / "head.safetensors", model.tensor_requests())


def test_random_weights_mode(tmp_path):
    a = tiny_configs.write_tiny("B", tmp_path / "a")
    b = tiny_configs.write_tiny("B", tmp_path / "b")
    assert json.loads((a / "config.json").read_text()) == tiny_configs.CONFIG_B
    ta, tb = plain_model.read_safetensors(a / "model.safetensors"), plain_model.read_safetensors(b / "model.safetensors")
    assert ta.keys() == tb.keys() and all(torch.equal(ta[k], tb[k]) for k in ta)          # same seed, same numbers
    c = write_random_model(tmp_path / "c", tiny_configs.CONFIG_B, seed=4, std=0.07, bias_std=0.1, gain_std=0.1,
                           store_dtype="float32")
    tc = plain_model.read_safetensors(c / "model.safetensors")
    assert not torch.equal(ta["lm_head.weight"], tc["lm_head.weight"])
    w = ta["model.layers.0.mlp.down_proj.weight"]
    assert w.shape == (80, 208) and abs(float(w.std()) - 0.07) < 0.005
    assert abs(float(ta["model.layers.1.self_attn.k_proj.bias"].std()) - 0.1) < 0.03
    g = ta["model.layers.2.input_layernorm.weight"]
    assert abs(float(g.mean()) - 1.0) < 0.05 and float(g.std()) > 0.05
    ones = plain_model.read_safetensors(tiny_configs.write_tiny("A", tmp_path / "d") / "model.safetensors")
    assert torch.equal(ones["model.norm.weight"], torch.ones(64))
    bf = write_random_model(tmp_path / "e", tiny_configs.CONFIG_A, seed=0, store_dtype="bfloat16")
    with SafetensorsFile(bf / "model.safetensors") as f:
        assert f.stored_dtype("model.embed_tokens.weight") == "BF16"
    with pytest.raises(ValueError):
        write_random_model(tmp_path / "f", {"architectures": ["Nope"]}, seed=0)
