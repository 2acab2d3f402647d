"""Configuration: typed parsing of config.json, refusals, and the architecture registry."""
from __future__ import annotations

import json
import os

import pytest

from helix_runtime_b200 import ConfigError, LlamaConfig, load_config, register_architecture
from helix_runtime_b200.config import architecture_for, known_architectures
from helix_runtime_b200.models import build_llama_spec
from tiny_configs import TINY_A, TINY_B, tiny_config


def document(**changes):
    base = tiny_config("A").to_dict()
    base.update(changes)
    return base


def test_round_trip_and_derived_fields(tmp_path):
    config = tiny_config("B")
    path = tmp_path / "config.json"
    path.write_text(json.dumps(config.to_dict()))
    architecture, loaded = load_config(str(tmp_path))
    assert architecture.name == "LlamaForCausalLM"
    assert loaded == config
    assert loaded.head_dim == 24 and loaded.num_key_value_heads == 5
    # defaults of the reference's converter: eps 1e-6, theta 1e4, heads for kv heads
    minimal = {k: v for k, v in config.to_dict().items()
               if k not in ("rms_norm_eps", "rope_theta", "num_key_value_heads", "head_dim")}
    parsed = LlamaConfig.from_dict(minimal)
    assert parsed.rms_norm_eps == 1e-6 and parsed.rope_theta == 10000.0
    assert parsed.num_key_value_heads == parsed.num_attention_heads
    assert parsed.head_dim == parsed.hidden_size // parsed.num_attention_heads


def test_the_two_tiny_configurations_differ_in_every_size():
    for key in TINY_A:
        assert TINY_A[key] != TINY_B[key], key


@pytest.mark.parametrize("changes,message", [
    (dict(model_type="mistral", architectures=["LlamaForCausalLM"]), "model_type"),
    (dict(num_key_value_heads=2), "num_key_value_heads"),
    (dict(head_dim=32), "head_dim"),
    (dict(hidden_size=66), "divisible"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(attention_bias=True), "biases"),
    (dict(mlp_bias=True), "biases"),
    (dict(rope_scaling={"type": "linear", "factor": 2.0}), "RoPE"),
    (dict(partial_rotary_factor=0.5), "partial rotary"),
    (dict(vocab_size=0), "vocab_size"),
    (dict(vocab_size=True), "vocab_size"),
    (dict(rms_norm_eps=-1.0), "rms_norm_eps"),
    (dict(rope_theta="big"), "rope_theta"),
    (dict(rope_parameters={"rope_type": "yarn"}), "default"),
    (dict(rope_parameters={"rope_theta": 5.0}), "disagree"),
    (dict(tie_word_embeddings="yes"), "tie_word_embeddings"),
])
def test_refusals(changes, message):
    with pytest.raises(ConfigError, match=message):
        LlamaConfig.from_dict(document(**changes))


def test_head_dim_must_be_even():
    with pytest.raises(ConfigError, match="even"):
        LlamaConfig.from_dict(document(hidden_size=60, num_attention_heads=4,
                                       num_key_value_heads=4, head_dim=15))


def test_duplicate_keys_and_bad_json_are_errors(tmp_path):
    (tmp_path / "config.json").write_text('{"model_type": "llama", "model_type": "llama"}')
    with pytest.raises(ConfigError, match="duplicate"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("[1, 2]")
    with pytest.raises(ConfigError, match="object"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{")
    with pytest.raises(ConfigError, match="parse"):
        load_config(str(tmp_path))


def test_registry_names_known_architectures_on_a_miss():
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):
        architecture_for({"architectures": ["NopeForCausalLM"], "model_type": "nope"})
    assert "LlamaForCausalLM" in known_architectures()
    # model_type alone is enough, as in the reference's converter
    assert architecture_for({"model_type": "llama"}).name == "LlamaForCausalLM"


def test_registering_another_architecture_needs_no_framework_change():
    calls = []

    def from_dict(doc):
        calls.append(doc)
        return LlamaConfig.from_dict({**doc, "model_type": "llama"})

    register_architecture("ToyForCausalLM", from_dict, build_llama_spec, aliases=("toy",))
    entry = architecture_for({"architectures": ["ToyForCausalLM"]})
    config = entry.config_from_dict(document(model_type="toy"))
    spec = entry.build_spec(config)
    assert len(spec.blocks) == 2 and calls
    with pytest.raises(ValueError, match="already registered"):
        register_architecture("OtherForCausalLM", from_dict, build_llama_spec, aliases=("toy",))


def test_spec_carries_every_size_as_a_parameter():
    config = tiny_config("B")
    spec = build_llama_spec(config)
    spec.validate()
    assert spec.hidden_size == 120 and spec.vocab_size == 384 and spec.max_positions == 256
    assert len(spec.blocks) == 3 and [entry.block for entry in spec.schedule] == [0, 1, 2]
    mixer = spec.blocks[1].mixer
    assert (mixer["num_heads"], mixer["num_kv_heads"], mixer["head_dim"]) == (5, 5, 24)
    assert mixer["position"]["theta"] == 500000.0 and mixer["position"]["pairing"] == "adjacent"
    assert spec.blocks[1].mixer_norm["eps"] == 1e-6
    assert spec.blocks[2].feed_forward["intermediate_size"] == 320
    assert mixer.tensors["q"] == "model.layers.1.self_attn.q_proj.weight"


def test_schedule_validation():
    import dataclasses
    from helix_runtime_b200.config import ScheduleEntry
    spec = build_llama_spec(tiny_config("A"))
    twice = dataclasses.replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1),
                                                ScheduleEntry(0), ScheduleEntry(1, cache_from=1)))
    twice.validate()
    with pytest.raises(ValueError, match="does not run before"):
        dataclasses.replace(spec, schedule=(ScheduleEntry(0, cache_from=1), ScheduleEntry(1))).validate()
    with pytest.raises(ValueError, match="names block"):
        dataclasses.replace(spec, schedule=(ScheduleEntry(5),)).validate()
    with pytest.raises(ValueError, match="owns none"):
        dataclasses.replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1, cache_from=0),
                                            ScheduleEntry(1, cache_from=1))).validate()
