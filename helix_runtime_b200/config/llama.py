"""Typed configuration of the Llama-style MHA decoder, read from ``config.json``.

Which keys are read, their defaults and what is refused follow the reference's checkpoint
converter (tools/convert_hf_llama.py:103-196) and its ``LlamaConfig::validate``
(src/model/llama.cpp:41-78): equal query and key/value heads, full adjacent-pair rotary
encoding without scaling, SiLU, no biases.  The keys are rows of a table
(:data:`LLAMA_KEYS`); the rules that tie several keys together are in ``validate``.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, Mapping

from .errors import ConfigError
from .keys import ABSENT, COUNT, FLAG, OBJECT, REAL, TEXT, Key, only_keys, read_keys

_SIZES = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
          "num_attention_heads", "max_position_embeddings")

LLAMA_KEYS = (
    Key("model_type", TEXT, requires="llama",
        refusal="config field 'model_type' must be exactly 'llama'"),
    *(Key(name, COUNT) for name in _SIZES),
    # absent or null: as many as there are query heads / hidden_size over heads
    Key("num_key_value_heads", COUNT, default=None, null_is_default=True),
    Key("head_dim", COUNT, default=None, null_is_default=True),
    Key("rms_norm_eps", REAL, default=1.0e-6),
    Key("rope_theta", REAL, default=10000.0),
    Key("tie_word_embeddings", FLAG, default=False),
    # what the kernels do not do: one value each, anything else is refused
    Key("hidden_act", TEXT, default="silu", requires="silu",
        refusal="only hidden_act='silu' is supported"),
    Key("attention_bias", FLAG, default=False, requires=False,
        refusal="attention projection biases are not supported"),
    Key("mlp_bias", FLAG, default=False, requires=False,
        refusal="MLP projection biases are not supported"),
    Key("partial_rotary_factor", REAL, default=1.0, requires=1.0,
        refusal="partial rotary dimensions are not supported"),
    Key("rope_scaling", ABSENT, default=None),
    Key("rope_parameters", OBJECT, default=None),
)

ROPE_PARAMETER_KEYS = (
    Key("rope_type", TEXT, default="default", requires="default",
        refusal="only default, unscaled RoPE is supported"),
    Key("partial_rotary_factor", REAL, default=1.0, requires=1.0,
        refusal="partial rotary dimensions are not supported"),
    Key("rope_theta", REAL, default=None),
)


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
        """Types of the fields (a configuration may be built in code, not only read) and
        the rules between them."""
        own = {field.name: getattr(self, field.name) for field in dataclasses.fields(self)}
        read_keys(own, [key for key in LLAMA_KEYS if key.name in own])
        heads, hidden = self.num_attention_heads, self.hidden_size
        if hidden % heads:
            raise ConfigError("hidden_size must be divisible by num_attention_heads")
        if self.head_dim != hidden // heads:
            raise ConfigError("head_dim must equal hidden_size / num_attention_heads")
        if self.head_dim % 2:
            raise ConfigError("the full rotary head dimension must be even")
        if self.num_key_value_heads != heads:
            raise ConfigError("num_key_value_heads must equal num_attention_heads; "
                              "GQA/MQA checkpoints are not this architecture")
        if self.vocab_size > 2 ** 32:
            raise ConfigError("vocab_size exceeds the 32-bit token id range")

    @classmethod
    def from_dict(cls, document: Mapping[str, Any]) -> "LlamaConfig":
        try:
            values = read_keys(document, LLAMA_KEYS)
        except ConfigError as problem:
            if "'rope_scaling'" in str(problem):
                raise ConfigError("scaled or dynamic RoPE configurations are not "
                                  "supported") from None
            raise
        heads, hidden = values["num_attention_heads"], values["hidden_size"]
        if hidden % heads:
            raise ConfigError("hidden_size must be divisible by num_attention_heads")
        if values["rope_parameters"] is not None:
            only_keys(values["rope_parameters"], ROPE_PARAMETER_KEYS, "rope_parameters")
            nested = read_keys(values["rope_parameters"], ROPE_PARAMETER_KEYS, "rope_parameters.")
            if nested["rope_theta"] not in (None, values["rope_theta"]):
                raise ConfigError("rope_theta and rope_parameters.rope_theta disagree")
        fields = {field.name for field in dataclasses.fields(cls)}
        chosen = {name: value for name, value in values.items() if name in fields}
        if chosen["num_key_value_heads"] is None:
            chosen["num_key_value_heads"] = heads
        if chosen["head_dim"] is None:
            chosen["head_dim"] = hidden // heads
        return cls(**chosen)

    def to_dict(self) -> Dict[str, Any]:
        document: Dict[str, Any] = {"architectures": [self.architecture],
                                    "model_type": self.model_type}
        document.update(dataclasses.asdict(self))
        document.update(hidden_act="silu", rope_scaling=None, attention_bias=False,
                        mlp_bias=False)
        return document

    def parameter_count(self) -> int:
        h, i, v = self.hidden_size, self.intermediate_size, self.vocab_size
        per_layer = 4 * h * h + 3 * h * i + 2 * h
        return v * h + self.num_hidden_layers * per_layer + h + (0 if self.tie_word_embeddings else v * h)
