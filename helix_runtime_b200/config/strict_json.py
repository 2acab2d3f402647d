"""JSON objects read strictly: a key that appears twice is an error, not a silent override.

Python's parser keeps the last of two equal keys; a configuration or a container header in
which a key is given twice is ambiguous, and the reference's tools refuse it
(tools/convert_hf_llama.py:43-49).  Both the configuration reader and the safetensors reader
parse through :func:`parse_object`, each with its own error class.
"""
from __future__ import annotations

import json
from typing import Any, Callable, Dict, Type, Union


def parse_object(text: Union[str, bytes], what: str,
                 error: Type[Exception] = ValueError) -> Dict[str, Any]:
    """Parse ``text`` as one JSON object; ``what`` names the source in messages."""
    repeated = []

    def collect(pairs):
        keys = [key for key, _ in pairs]
        repeated.extend(key for key in set(keys) if keys.count(key) > 1)
        return dict(pairs)

    try:
        if isinstance(text, bytes):
            text = text.decode("utf-8")
        document = json.loads(text, object_pairs_hook=collect)
    except (UnicodeError, json.JSONDecodeError) as problem:
        raise error(f"{what}: invalid JSON: {problem}") from problem
    if repeated:
        raise error(f"{what}: JSON object contains duplicate key {sorted(repeated)[0]!r}")
    if not isinstance(document, dict):
        raise error(f"{what}: the JSON root must be an object")
    return document
