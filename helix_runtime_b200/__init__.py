"""helix_runtime_b200: a small, whole, single-GPU inference engine for NVIDIA B200.

It serves one architecture, the Llama-style decoder with equal query and key/value
heads that ``parthpandya5/helix-runtime`` runs (src/model/cpu_llama.cpp), from a
model folder (``config.json`` + safetensors) to generated tokens:

>>> from helix_runtime_b200 import Engine
>>> engine = Engine.from_pretrained("/path/to/model", dtype="bfloat16")
>>> engine.generate([[1, 42, 17]], max_new_tokens=8)[0].generated_tokens
"""
from . import models  # noqa: F401  (registers the architecture and the parts)
from .models import register_arrangement
from .config import (ConfigError, LlamaConfig, ModelSpec, PartSpec, load_config,
                     register_architecture)
from .engine import (Engine, EngineConfig, GenerationResult, StepEntry, StepError, StepFunction,
                     load_model, random_model, write_random_model)
from .parts import register_part
from .weights import WeightError

__version__ = "0.1.0"

__all__ = [
    "ConfigError", "Engine", "EngineConfig", "GenerationResult", "LlamaConfig", "ModelSpec",
    "PartSpec", "StepEntry", "StepError", "StepFunction", "WeightError", "load_config",
    "load_model", "random_model", "register_architecture", "register_arrangement",
    "register_part",
    "write_random_model",
]
