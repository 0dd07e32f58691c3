"""Weights: the safetensors reader's refusals, the one error for tensors that do not fit, the random-weights mode."""
import json
import os
import struct

import pytest
import torch

from configs import TINY_A, TINY_B
from llmx_b200.config import Qwen3Config
from llmx_b200.registry import architecture_of
from llmx_b200.weights import (RandomSource, SafetensorsError, TensorDirectory, WeightError, check_tensors, read_header,
                               write_random_model, write_safetensors)


def _raw_file(path, header, data=b""):
    text = json.dumps(header).encode() if not isinstance(header, bytes) else header
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + data)


def test_round_trip_keeps_storage_types(tmp_path):
    tensors = {"a": torch.arange(6, dtype=torch.float32).view(2, 3), "b": torch.ones(4, dtype=torch.bfloat16),
               "c": torch.tensor([[1, -2]], dtype=torch.int64), "d": torch.zeros(0, 5, dtype=torch.float16)}
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, tensors, {"k": "v"})
    entries, meta = read_header(p)
    assert meta == {"k": "v"} and set(entries) == set(tensors)
    d = TensorDirectory(str(tmp_path))
    for n, t in tensors.items():
        assert d.dtype(n) == t.dtype and d.shape(n) == tuple(t.shape) and torch.equal(d.tensor(n), t)
    # The same file through the safetensors library: the writer follows the format.
    from safetensors.torch import load_file
    back = load_file(p)
    assert all(torch.equal(back[n], t) for n, t in tensors.items())


@pytest.mark.parametrize("make,message", [
    (lambda p: open(p, "wb").write(b"abc"), "shorter than a safetensors header"),
    (lambda p: open(p, "wb").write(struct.pack("<Q", 1 << 40)), "exceeds"),
    (lambda p: open(p, "wb").write(struct.pack("<Q", 100) + b"{}"), "past the end"),
    (lambda p: _raw_file(p, b"[1, 2]"), "not a JSON object"),
    (lambda p: _raw_file(p, b"{not json"), "not JSON"),
    (lambda p: _raw_file(p, b'{"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}, "a": {"dtype": "F32", "shape": [1], "data_offsets": [4, 8]}}', b"\0" * 8), "repeats the key"),
    (lambda p: _raw_file(p, {"a": {"dtype": "F32", "shape": [1]}}), "exactly dtype, shape and data_offsets"),
    (lambda p: _raw_file(p, {"a": {"dtype": "F99", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 4), "unsupported dtype"),
    (lambda p: _raw_file(p, {"a": {"dtype": "F32", "shape": [1, 1, 1, 1, 1, 1], "data_offsets": [0, 4]}}, b"\0" * 4), "invalid shape"),
    (lambda p: _raw_file(p, {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 4), "offsets span"),
    (lambda p: _raw_file(p, {"a": {"dtype": "F32", "shape": [1], "data_offsets": [4, 8]}}, b"\0" * 8), "leaves a gap"),
    (lambda p: _raw_file(p, {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}, "b": {"dtype": "F32", "shape": [1], "data_offsets": [4, 8]}}, b"\0" * 8), "overlaps"),
    (lambda p: _raw_file(p, {"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 9), "the file at"),
])
def test_file_refusals(tmp_path, make, message):
    p = str(tmp_path / "model.safetensors")
    make(p)
    with pytest.raises(SafetensorsError) as e:
        read_header(p)
    assert message in str(e.value)


def test_index_file(tmp_path):
    write_safetensors(str(tmp_path / "one.safetensors"), {"a": torch.ones(2)})
    write_safetensors(str(tmp_path / "two.safetensors"), {"b": torch.zeros(3)})
    idx = tmp_path / "model.safetensors.index.json"
    idx.write_text(json.dumps({"weight_map": {"a": "one.safetensors", "b": "two.safetensors"}}))
    d = TensorDirectory(str(tmp_path))
    assert sorted(d.names()) == ["a", "b"] and d.tensor("b").shape == (3,)
    idx.write_text(json.dumps({"weight_map": {"a": "one.safetensors", "b": "one.safetensors"}}))
    with pytest.raises(SafetensorsError, match="disagree"):
        TensorDirectory(str(tmp_path))
    idx.write_text(json.dumps({"weight_map": {"a": "../one.safetensors"}}))
    with pytest.raises(SafetensorsError, match="outside the model folder"):
        TensorDirectory(str(tmp_path))
    idx.unlink()
    with pytest.raises(SafetensorsError, match="neither"):
        TensorDirectory(str(tmp_path))


def _model(raw):
    cfg = Qwen3Config.from_dict(raw)
    return cfg, architecture_of(cfg.to_dict()).build(cfg)


def test_expected_tensors_of_the_architecture():
    cfg, model = _model(TINY_B)
    specs = model.tensor_specs()
    assert len(specs) == 3 + 3 * 11
    assert specs["model.embed_tokens.weight"].shape == (384, 96) and specs["lm_head.weight"].shape == (384, 96)
    assert specs["model.layers.2.self_attn.q_proj.weight"].shape == (192, 96)
    assert specs["model.layers.0.self_attn.k_norm.weight"].shape == (32,)
    assert specs["model.layers.1.mlp.down_proj.weight"].shape == (96, 160)
    _, tied = _model(TINY_A)
    assert "lm_head.weight" not in tied.tensor_specs() and "lm_head.weight" in tied.ignorable


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    cfg, model = _model(TINY_A)
    src = RandomSource(model.tensor_specs(), 0, dtype=torch.float32)
    tensors = {n: src.tensor(n) for n in src.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.7.mlp.up_proj.weight"] = torch.zeros(2, 2)
    tensors["rotary.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63)
    tensors["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        check_tensors(model.tensor_specs(), TensorDirectory(str(tmp_path)), "here", model.ignorable)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.7.mlp.up_proj.weight", "rotary.inv_freq"]
    assert [n for n, _ in err.wrong] == ["model.layers.0.input_layernorm.weight", "model.layers.0.self_attn.q_proj.weight"]
    text = str(err)
    assert "missing (2)" in text and "unexpected (2)" in text and "shape [64, 63], expected [64, 64]" in text


def test_tied_model_ignores_a_stored_head_and_untied_needs_one(tmp_path):
    cfg, model = _model(TINY_A)
    src = RandomSource(model.tensor_specs(), 0)
    tensors = {n: src.tensor(n) for n in src.names()}
    tensors["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    check_tensors(model.tensor_specs(), TensorDirectory(str(tmp_path)), "tied", model.ignorable)
    untied_cfg, untied = _model(dict(TINY_A, tie_word_embeddings=False))
    del tensors["lm_head.weight"]
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        check_tensors(untied.tensor_specs(), TensorDirectory(str(tmp_path)), "untied", untied.ignorable)
    assert e.value.missing == ["lm_head.weight"]


def test_random_weights_mode_writes_a_model_folder(tmp_path):
    cfg, model = _model(TINY_B)
    d = write_random_model(str(tmp_path / "m"), cfg, seed=5)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    assert Qwen3Config.from_dict(json.load(open(os.path.join(d, "config.json")))) == cfg
    t = TensorDirectory(d)
    check_tensors(model.tensor_specs(), t, d, model.ignorable)
    emb = t.tensor("model.embed_tokens.weight").float()
    norm = t.tensor("model.layers.0.input_layernorm.weight")
    assert t.dtype("model.embed_tokens.weight") == torch.bfloat16 and norm.dtype == torch.float32   # a 32-bit tensor stays so
    assert abs(emb.std().item() - 0.02) < 0.002 and abs(emb.mean().item()) < 0.001
    assert abs(norm.mean().item() - 1.0) < 0.01 and 0.005 < norm.std().item() < 0.02
    # The same seed gives the same folder; another seed another; a tensor does not depend on the others.
    d2 = write_random_model(str(tmp_path / "m2"), cfg, seed=5)
    d3 = write_random_model(str(tmp_path / "m3"), cfg, seed=6)
    assert torch.equal(TensorDirectory(d2).tensor("lm_head.weight"), t.tensor("lm_head.weight"))
    assert not torch.equal(TensorDirectory(d3).tensor("lm_head.weight"), t.tensor("lm_head.weight"))
    only = RandomSource({"lm_head.weight": model.tensor_specs()["lm_head.weight"]}, 5)
    assert torch.equal(only.tensor("lm_head.weight"), t.tensor("lm_head.weight"))


def test_random_values_are_a_function_of_seed_name_and_index():
    """The generator is counter-based: a tensor's values depend on (seed, name, element index) alone -- not on how the
    work is cut into chunks, on the other tensors, or on the order of making them -- and look like N(0, 1)."""
    import torch
    from llmx_b200.weights.random_init import RandomSource, standard_normal
    from llmx_b200.weights.spec import TensorSpec
    cpu = torch.device("cpu")
    x = standard_normal(99, 200_000, cpu)
    assert torch.equal(x[:5000], standard_normal(99, 5000, cpu, chunk=777))
    assert abs(float(x.mean())) < 0.01 and abs(float(x.std()) - 1.0) < 0.01 and float(x.abs().max()) < 5.5
    assert abs(float(((x[:-1] * x[1:]).mean()))) < 0.01                      # neighbours are not correlated
    assert not torch.equal(x[:100], standard_normal(100, 100, cpu))
    specs = {"a.weight": TensorSpec((6, 10)), "b.weight": TensorSpec((10,), "vector", init="one_plus_normal", std=0.01)}
    one = RandomSource(specs, 3, dtype=torch.float32)
    other = RandomSource({"b.weight": specs["b.weight"]}, 3, dtype=torch.float32)
    assert torch.equal(one.tensor("b.weight"), other.tensor("b.weight"))
    assert abs(float(one.tensor("b.weight").mean()) - 1.0) < 0.02
    assert not torch.equal(one.tensor("a.weight"), RandomSource(specs, 4, dtype=torch.float32).tensor("a.weight"))
