"""``config.json`` keys as data: a table says what a key holds, its default, and which value
the engine requires of it; one function walks a table over a document.

An architecture's configuration class lists its keys once (see ``config/llama.py``) instead of
writing a check per key, and a key that a model must not set to anything but one value (an
activation that has no kernel, a bias that no kernel adds) is a row with ``requires``.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Callable, Dict, Mapping, Optional, Sequence

from .errors import ConfigError

REQUIRED = object()       # no default: the key must be there
ANYTHING = object()       # no required value


def _count(value: Any) -> bool:
    return isinstance(value, int) and not isinstance(value, bool) and value > 0


def _real(value: Any) -> bool:
    return (isinstance(value, (int, float)) and not isinstance(value, bool)
            and math.isfinite(float(value)) and float(value) > 0.0)


@dataclasses.dataclass(frozen=True)
class Kind:
    accepts: Callable[[Any], bool]
    convert: Callable[[Any], Any]
    complaint: str


COUNT = Kind(_count, int, "must be a positive integer")
REAL = Kind(_real, float, "must be a positive, finite number")
FLAG = Kind(lambda value: isinstance(value, bool), bool, "must be a boolean")
TEXT = Kind(lambda value: isinstance(value, str), str, "must be a string")
OBJECT = Kind(lambda value: isinstance(value, dict), dict, "must be an object")
ABSENT = Kind(lambda value: value is None, lambda value: None, "must be null")


@dataclasses.dataclass(frozen=True)
class Key:
    name: str
    kind: Kind
    default: Any = REQUIRED
    requires: Any = ANYTHING          # the one value this engine runs
    refusal: Optional[str] = None     # what to say when ``requires`` is not met
    null_is_default: bool = False     # an explicit null stands for the default


def read_keys(document: Mapping[str, Any], table: Sequence[Key], prefix: str = "") -> Dict[str, Any]:
    """The table's keys out of ``document``: typed, defaulted, checked against ``requires``."""
    values: Dict[str, Any] = {}
    for key in table:
        label = f"config field {prefix + key.name!r}"
        raw = document.get(key.name, key.default)
        if raw is None and key.null_is_default:
            raw = key.default
        unset = raw is None and key.default is None          # an optional key left out
        if raw is REQUIRED or not (unset or key.kind.accepts(raw)):
            raise ConfigError(f"{label} {key.kind.complaint}")
        value = None if raw is None else key.kind.convert(raw)
        if key.requires is not ANYTHING and value != key.requires:
            raise ConfigError(key.refusal or f"{label} must be {key.requires!r}")
        values[key.name] = value
    return values


def only_keys(document: Mapping[str, Any], table: Sequence[Key], what: str) -> None:
    unknown = sorted(set(document) - {key.name for key in table})
    if unknown:
        raise ConfigError(f"unsupported {what} fields: {', '.join(unknown)}")
