"""One registry from an architecture's name to its configuration class and model spec.

``config.json`` chooses the model everywhere in the engine: ``architectures[0]``
is looked up first, then ``model_type``.  The reference has only the gate
``model_type == "llama"`` (tools/convert_hf_llama.py:105-106) and a model-kind
code in its file header (src/model/format.cpp:44); the registry generalises that
gate so a second architecture is one ``register_architecture`` call.
"""
from __future__ import annotations

import dataclasses
import os
from typing import Any, Callable, Dict, Mapping, Tuple

from .errors import ConfigError
from .strict_json import parse_object
from .spec import ModelSpec


@dataclasses.dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[Mapping[str, Any]], Any]
    build_spec: Callable[[Any], ModelSpec]
    aliases: Tuple[str, ...] = ()


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_from_dict: Callable[[Mapping[str, Any]], Any],
                          build_spec: Callable[[Any], ModelSpec],
                          aliases: Tuple[str, ...] = ()) -> Architecture:
    """Register ``name`` (the string in ``config.json``'s ``architectures``).

    ``config_from_dict`` turns the parsed JSON object into a typed configuration
    (raising :class:`ConfigError`), ``build_spec`` turns that configuration into
    the part-by-part :class:`ModelSpec`.  ``aliases`` are ``model_type`` values.
    """
    entry = Architecture(name, config_from_dict, build_spec, tuple(aliases))
    for key in (name, *aliases):
        existing = _ARCHITECTURES.get(key)
        if existing is not None and existing.name != name:
            raise ValueError(f"architecture key {key!r} is already registered to {existing.name!r}")
        _ARCHITECTURES[key] = entry
    return entry


def known_architectures() -> Tuple[str, ...]:
    return tuple(sorted({entry.name for entry in _ARCHITECTURES.values()}))


def architecture_for(document: Mapping[str, Any]) -> Architecture:
    names = document.get("architectures")
    candidates = []
    if isinstance(names, list):
        candidates.extend(name for name in names if isinstance(name, str))
    model_type = document.get("model_type")
    if isinstance(model_type, str):
        candidates.append(model_type)
    for candidate in candidates:
        entry = _ARCHITECTURES.get(candidate)
        if entry is not None:
            return entry
    raise ConfigError(
        f"no registered architecture for architectures={names!r} model_type={model_type!r}; "
        f"known: {', '.join(known_architectures()) or '(none)'}")


def read_config_json(path: str) -> Dict[str, Any]:
    """``config.json`` as a dictionary; a key given twice, a root that is no object and text
    that is no JSON are errors (tools/convert_hf_llama.py:43-49)."""
    try:
        with open(path, "rb") as source:
            text = source.read()
    except OSError as problem:
        raise ConfigError(f"could not parse {path}: {problem}") from problem
    return parse_object(text, f"could not parse {path}", ConfigError)


def load_config(model_dir: str):
    """Return ``(architecture, typed config)`` for a model folder."""
    document = read_config_json(os.path.join(model_dir, "config.json"))
    entry = architecture_for(document)
    return entry, entry.config_from_dict(document)
