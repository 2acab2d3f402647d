"""Weights: the safetensors container, loading by name with one error for everything wrong,
dtype policy, and the random-weights mode."""
from __future__ import annotations

import json
import os
import struct

import numpy as np
import pytest
import torch

from helix_runtime_b200 import WeightError, load_model, write_random_model
from helix_runtime_b200.weights import (Checkpoint, SafetensorsError, TensorRequest,
                                        load_tensors, write_safetensors)
from tiny_configs import make_folder, tiny_config


def test_container_round_trip(tmp_path):
    tensors = {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3),
               "b": torch.randn(5).to(torch.bfloat16),
               "c": torch.tensor([1, 2, 3], dtype=torch.int32),
               "d": torch.randn(2, 2).to(torch.float16)}
    path = tmp_path / "model.safetensors"
    write_safetensors(str(path), tensors)
    checkpoint = Checkpoint(str(tmp_path))
    assert sorted(checkpoint.names()) == ["a", "b", "c", "d"]
    for name, tensor in tensors.items():
        assert torch.equal(checkpoint.read(name), tensor)
    # the installed safetensors package reads the same bytes
    from safetensors.torch import load_file
    for name, tensor in load_file(str(path)).items():
        assert torch.equal(tensor, tensors[name])


def corrupt(tmp_path, mutate):
    tensors = {"a": torch.zeros(4), "b": torch.ones(2)}
    path = tmp_path / "model.safetensors"
    write_safetensors(str(path), tensors)
    raw = path.read_bytes()
    (length,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + length])
    payload = raw[8 + length:]
    header, payload = mutate(header, payload)
    encoded = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(encoded)) + encoded + payload)
    return str(tmp_path)


@pytest.mark.parametrize("mutate,message", [
    (lambda h, p: ({**h, "a": {**h["a"], "data_offsets": [0, 12]}}, p), "byte range"),
    (lambda h, p: ({**h, "b": {**h["b"], "data_offsets": [8, 16]}}, p), "overlaps"),
    (lambda h, p: (h, p + b"\0\0\0\0"), "trailing"),
    (lambda h, p: ({**h, "a": {**h["a"], "dtype": "F8"}}, p), "unsupported dtype"),
    (lambda h, p: ({**h, "a": {**h["a"], "extra": 1}}, p), "noncanonical"),
    (lambda h, p: ({**h, "b": {**h["b"], "data_offsets": [16, 30]}}, p), "bounds"),
])
def test_malformed_containers_are_refused(tmp_path, mutate, message):
    folder = corrupt(tmp_path, mutate)
    with pytest.raises(SafetensorsError, match=message):
        Checkpoint(folder)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path, model_root):
    folder = make_folder(model_root, "A", storage_dtype="float32")
    checkpoint = Checkpoint(folder)
    tensors = {name: checkpoint.read(name) for name in checkpoint.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(64, 32)
    tensors["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.int32)
    broken = tmp_path / "broken"
    broken.mkdir()
    (broken / "config.json").write_text(json.dumps(tiny_config("A").to_dict()))
    write_safetensors(str(broken / "model.safetensors"), tensors)
    with pytest.raises(WeightError) as caught:
        load_model(str(broken), "float32", "cpu")
    error = caught.value
    assert error.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert error.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert error.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (64, 32), (64, 64))]
    text = str(error)
    for fragment in ("missing tensors (2)", "unexpected tensors (1)", "q_proj.bias",
                     "is [64, 32], expected [64, 64]", "lm_head.weight is stored as I32"):
        assert fragment in text


def test_non_finite_weights_are_refused(tmp_path, model_root):
    folder = make_folder(model_root, "A", storage_dtype="float32")
    checkpoint = Checkpoint(folder)
    tensors = {name: checkpoint.read(name) for name in checkpoint.names()}
    tensors["model.layers.0.mlp.down_proj.weight"][3, 3] = float("nan")
    bad = tmp_path / "nan"
    bad.mkdir()
    (bad / "config.json").write_text(json.dumps(tiny_config("A").to_dict()))
    write_safetensors(str(bad / "model.safetensors"), tensors)
    with pytest.raises(WeightError, match="non-finite values in model.layers.0.mlp.down_proj"):
        load_model(str(bad), "float32", "cpu")


def test_dtype_policy(tmp_path):
    tensors = {"matrix16": torch.randn(4, 8).to(torch.bfloat16), "matrix32": torch.randn(4, 8),
               "scale16": torch.randn(8).to(torch.bfloat16), "scale32": torch.randn(8),
               "table": torch.arange(5, dtype=torch.int64)}
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    requests = [TensorRequest("matrix16", (4, 8)), TensorRequest("matrix32", (4, 8)),
                TensorRequest("scale16", (8,), role="scale"),
                TensorRequest("scale32", (8,), role="scale"),
                TensorRequest("table", (5,), role="table")]
    checkpoint = Checkpoint(str(tmp_path))
    served = load_tensors(checkpoint, requests, torch.bfloat16, torch.device("cpu"))
    assert served["matrix16"].dtype == torch.bfloat16 and served["matrix32"].dtype == torch.bfloat16
    assert torch.equal(served["matrix16"], tensors["matrix16"])            # kept as stored
    assert served["scale32"].dtype == torch.float32 and torch.equal(served["scale32"], tensors["scale32"])
    assert served["scale16"].dtype == torch.float32
    assert torch.equal(served["scale16"], tensors["scale16"].float())       # widened exactly
    assert served["table"].dtype == torch.int32
    true32 = load_tensors(checkpoint, requests, torch.float32, torch.device("cpu"))
    assert all(true32[name].dtype == torch.float32 for name in ("matrix16", "matrix32", "scale16"))


def test_tied_head_falls_back_to_the_embedding(tmp_path, model_root):
    import dataclasses
    folder = make_folder(model_root, "A", storage_dtype="float32")
    checkpoint = Checkpoint(folder)
    tensors = {name: checkpoint.read(name) for name in checkpoint.names() if name != "lm_head.weight"}
    tied = tmp_path / "tied"
    tied.mkdir()
    config = dataclasses.replace(tiny_config("A"), tie_word_embeddings=True)
    (tied / "config.json").write_text(json.dumps(config.to_dict()))
    write_safetensors(str(tied / "model.safetensors"), tensors)
    model = load_model(str(tied), "float32", "cpu")
    assert torch.equal(model.lm_head.weight.matrix, model.embedding.table)
    untied = tmp_path / "untied"
    untied.mkdir()
    (untied / "config.json").write_text(json.dumps(tiny_config("A").to_dict()))
    write_safetensors(str(untied / "model.safetensors"), tensors)
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_model(str(untied), "float32", "cpu")


def test_random_weights_mode_is_seeded_and_complete(tmp_path):
    config = tiny_config("B")
    write_random_model(str(tmp_path / "one"), config, seed=5)
    write_random_model(str(tmp_path / "two"), config, seed=5)
    write_random_model(str(tmp_path / "three"), config, seed=6)
    one, two, three = (Checkpoint(str(tmp_path / name)) for name in ("one", "two", "three"))
    assert sorted(os.listdir(tmp_path / "one")) == ["config.json", "model.safetensors"]
    assert len(one.names()) == 3 + 9 * config.num_hidden_layers
    name = "model.layers.2.mlp.gate_proj.weight"
    assert one.record(name).dtype == "BF16" and one.record(name).shape == (320, 120)
    assert torch.equal(one.read(name), two.read(name))
    assert not torch.equal(one.read(name), three.read(name))
    values = one.read(name).float()
    assert abs(float(values.std()) - 0.02) < 0.002 and abs(float(values.mean())) < 0.002
    assert torch.equal(one.read("model.norm.weight"), torch.ones(120))
    assert one.record("model.norm.weight").dtype == "F32"
    model = load_model(str(tmp_path / "one"), "bfloat16", "cpu")
    # five heads of 24, each held in a row of 32 (the next multiple of 16)
    assert model.blocks[0].mixer.w_qkv.shape == (3 * 5 * 32, 120)
    assert model.blocks[0].feed_forward.w_gate_up.shape == (640, 120)
    assert model.final_norm.weight.dtype == torch.float32


def test_rotary_row_permutation_matches_the_plain_conversion(model_root):
    import plain_llama
    folder = make_folder(model_root, "B", storage_dtype="float32")
    model = load_model(folder, "float32", "cpu")
    plain = plain_llama.PlainModel(folder)
    # [q | k | v] x five heads, each head's 24 rows followed by 8 rows of zeros
    fused = model.blocks[1].mixer.w_qkv.matrix.numpy().reshape(3, 5, 32, 120)
    assert not fused[:, :, 24:].any()
    for index, name in enumerate(("query", "key", "value")):
        np.testing.assert_array_equal(fused[index, :, :24].reshape(120, 120),
                                      plain.weights[f"layer.1.{name}"].T)
    out = model.blocks[1].mixer.w_o.matrix.numpy().reshape(120, 5, 32)
    assert not out[:, :, 24:].any()
    np.testing.assert_array_equal(out[:, :, :24].reshape(120, 120),
                                  plain.weights["layer.1.attention_output"].T)


def test_sharded_checkpoints_resolve_inside_the_folder_only(tmp_path):
    """An index maps tensor names to shard files (tools/convert_hf_llama.py:316-368)."""
    folder = tmp_path / "sharded"
    folder.mkdir()
    write_safetensors(str(folder / "one.safetensors"), {"a": torch.arange(4.0)})
    write_safetensors(str(folder / "two.safetensors"), {"b": torch.ones(2, 2), "c": torch.zeros(3)})
    index = {"metadata": {}, "weight_map": {"a": "one.safetensors", "b": "two.safetensors",
                                            "c": "two.safetensors"}}
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    checkpoint = Checkpoint(str(folder))
    assert sorted(checkpoint.names()) == ["a", "b", "c"]
    assert torch.equal(checkpoint.read("a"), torch.arange(4.0))
    assert checkpoint.record("b").shape == (2, 2)
    # a shard that lacks the tensor the index gives it
    index["weight_map"]["c"] = "one.safetensors"
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(SafetensorsError, match="lacks it"):
        Checkpoint(str(folder))
    # a shard outside the folder, by a relative path or a link
    write_safetensors(str(tmp_path / "outside.safetensors"), {"c": torch.zeros(3)})
    index["weight_map"]["c"] = "../outside.safetensors"
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(SafetensorsError, match="does not resolve inside"):
        Checkpoint(str(folder))
    os.symlink(str(tmp_path / "outside.safetensors"), str(folder / "link.safetensors"))
    index["weight_map"]["c"] = "link.safetensors"
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(SafetensorsError, match="does not resolve inside"):
        Checkpoint(str(folder))
    # a key given twice in the index
    (folder / "model.safetensors.index.json").write_text(
        '{"weight_map": {"a": "one.safetensors"}, "weight_map": {}}')
    with pytest.raises(SafetensorsError, match="duplicate key 'weight_map'"):
        Checkpoint(str(folder))
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(SafetensorsError, match="contains neither"):
        Checkpoint(str(empty))
