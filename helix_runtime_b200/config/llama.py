"""Typed configuration of the Llama-style MHA decoder, read from ``config.json``.

Keys, defaults and refusals follow the reference's checkpoint converter
(tools/convert_hf_llama.py:103-196) and its C++ ``LlamaConfig::validate``
(src/model/llama.cpp:41-78): equal query and key/value heads, full adjacent-pair
rotary encoding without scaling, SiLU, no biases.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Dict, Mapping

from .errors import ConfigError


def _positive_int(document: Mapping[str, Any], name: str) -> int:
    value = document.get(name)
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config field {name!r} must be a positive integer")
    return value


def _optional_bool(document: Mapping[str, Any], name: str, default: bool) -> bool:
    value = document.get(name, default)
    if not isinstance(value, bool):
        raise ConfigError(f"config field {name!r} must be a boolean")
    return value


def _positive_finite(value: Any, name: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config field {name!r} must be a number")
    result = float(value)
    if not math.isfinite(result) or result <= 0.0:
        raise ConfigError(f"config field {name!r} must be positive and finite")
    return result


@dataclasses.dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    max_position_embeddings: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float = 1.0e-6
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False

    model_type = "llama"
    architecture = "LlamaForCausalLM"

    def __post_init__(self) -> None:
        self.validate()

    def validate(self) -> None:
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "max_position_embeddings", "num_key_value_heads",
                     "head_dim"):
            value = getattr(self, name)
            if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
                raise ConfigError(f"config field {name!r} must be a positive integer")
        if self.hidden_size % self.num_attention_heads != 0:
            raise ConfigError("hidden_size must be divisible by num_attention_heads")
        if self.head_dim != self.hidden_size // self.num_attention_heads:
            raise ConfigError("head_dim must equal hidden_size / num_attention_heads")
        if self.head_dim % 2 != 0:
            raise ConfigError("the full rotary head dimension must be even")
        if self.num_key_value_heads != self.num_attention_heads:
            raise ConfigError(
                "num_key_value_heads must equal num_attention_heads; "
                "GQA/MQA checkpoints are not this architecture")
        if self.vocab_size > 2 ** 32:
            raise ConfigError("vocab_size exceeds the 32-bit token id range")
        _positive_finite(self.rms_norm_eps, "rms_norm_eps")
        _positive_finite(self.rope_theta, "rope_theta")
        if not isinstance(self.tie_word_embeddings, bool):
            raise ConfigError("config field 'tie_word_embeddings' must be a boolean")

    @classmethod
    def from_dict(cls, document: Mapping[str, Any]) -> "LlamaConfig":
        if document.get("model_type") != "llama":
            raise ConfigError("config field 'model_type' must be exactly 'llama'")
        vocab = _positive_int(document, "vocab_size")
        hidden = _positive_int(document, "hidden_size")
        intermediate = _positive_int(document, "intermediate_size")
        layers = _positive_int(document, "num_hidden_layers")
        heads = _positive_int(document, "num_attention_heads")
        max_positions = _positive_int(document, "max_position_embeddings")
        if hidden % heads != 0:
            raise ConfigError("hidden_size must be divisible by num_attention_heads")
        derived_head_dim = hidden // heads

        kv_heads = document.get("num_key_value_heads", heads)
        if kv_heads is None:
            kv_heads = heads
        if isinstance(kv_heads, bool) or not isinstance(kv_heads, int):
            raise ConfigError("config field 'num_key_value_heads' must be an integer")
        head_dim = document.get("head_dim", derived_head_dim)
        if head_dim is None:
            head_dim = derived_head_dim
        if isinstance(head_dim, bool) or not isinstance(head_dim, int):
            raise ConfigError("config field 'head_dim' must be an integer")

        if document.get("hidden_act", "silu") != "silu":
            raise ConfigError("only hidden_act='silu' is supported")
        if _optional_bool(document, "attention_bias", False):
            raise ConfigError("attention projection biases are not supported")
        if _optional_bool(document, "mlp_bias", False):
            raise ConfigError("MLP projection biases are not supported")
        if _positive_finite(document.get("partial_rotary_factor", 1.0),
                            "partial_rotary_factor") != 1.0:
            raise ConfigError("partial rotary dimensions are not supported")
        if document.get("rope_scaling") is not None:
            raise ConfigError("scaled or dynamic RoPE configurations are not supported")

        parameter_theta = None
        rope_parameters = document.get("rope_parameters")
        if rope_parameters is not None:
            if not isinstance(rope_parameters, dict):
                raise ConfigError("config field 'rope_parameters' must be an object")
            unknown = set(rope_parameters) - {"rope_type", "rope_theta", "partial_rotary_factor"}
            if unknown:
                raise ConfigError("unsupported rope_parameters fields: "
                                  + ", ".join(sorted(unknown)))
            if rope_parameters.get("rope_type", "default") != "default":
                raise ConfigError("only default, unscaled RoPE is supported")
            if _positive_finite(rope_parameters.get("partial_rotary_factor", 1.0),
                                "rope_parameters.partial_rotary_factor") != 1.0:
                raise ConfigError("partial rotary dimensions are not supported")
            if "rope_theta" in rope_parameters:
                parameter_theta = _positive_finite(rope_parameters["rope_theta"],
                                                   "rope_parameters.rope_theta")
        theta = _positive_finite(document.get("rope_theta", 10000.0), "rope_theta")
        if parameter_theta is not None and parameter_theta != theta:
            raise ConfigError("rope_theta and rope_parameters.rope_theta disagree")

        return cls(
            vocab_size=vocab,
            hidden_size=hidden,
            intermediate_size=intermediate,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            max_position_embeddings=max_positions,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=_positive_finite(document.get("rms_norm_eps", 1.0e-6), "rms_norm_eps"),
            rope_theta=theta,
            tie_word_embeddings=_optional_bool(document, "tie_word_embeddings", False),
        )

    def to_dict(self) -> Dict[str, Any]:
        return {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "attention_bias": False,
            "mlp_bias": False,
            "tie_word_embeddings": self.tie_word_embeddings,
        }

    def parameter_count(self) -> int:
        h, i, v = self.hidden_size, self.intermediate_size, self.vocab_size
        per_layer = 4 * h * h + 3 * h * i + 2 * h
        return v * h + self.num_hidden_layers * per_layer + h + (0 if self.tie_word_embeddings else v * h)
