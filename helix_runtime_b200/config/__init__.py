from .errors import ConfigError
from .llama import LlamaConfig
from .registry import (Architecture, architecture_for, known_architectures, load_config,
                       read_config_json, register_architecture)
from .spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry

__all__ = [
    "Architecture", "BlockSpec", "ConfigError", "LlamaConfig", "ModelSpec", "PartSpec",
    "ScheduleEntry", "architecture_for", "known_architectures", "load_config",
    "read_config_json", "register_architecture",
]
