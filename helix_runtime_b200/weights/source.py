"""Where a model comes from: a folder (``config.json`` + safetensors) or a Helix model file.

Both give the same two things: the configuration document that chooses the architecture, and
a weight source with ``names() / record(name) / read(name)`` in the checkpoint's names and
layout.  The reference's command line takes its native file
(examples/generate.cpp:22-27); its converter reads the folder
(tools/convert_hf_llama.py:656-716).
"""
from __future__ import annotations

import os
from typing import Any, Dict, Tuple

from ..config.errors import ConfigError
from ..config.registry import read_config_json
from .helix_file import HelixFile, is_helix_file
from .safetensors_io import Checkpoint


def open_model(path: str) -> Tuple[Dict[str, Any], Any]:
    """``(configuration document, weight source)`` for a model folder or a ``.helix`` file."""
    if os.path.isdir(path):
        return read_config_json(os.path.join(path, "config.json")), Checkpoint(path)
    if is_helix_file(path):
        source = HelixFile(path)
        return source.config_document(), source
    if os.path.isfile(path):
        # not the magic: let the reader say what is wrong with it
        HelixFile(path)
    raise ConfigError(f"{path} is neither a model folder (config.json, model.safetensors) "
                      "nor a Helix model file")
