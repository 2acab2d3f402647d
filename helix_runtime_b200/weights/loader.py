"""Load tensors by name, check them all, and report every problem in one error.

The reference validates a weight bundle tensor by tensor (src/model/llama.cpp:94-126)
and its converter refuses missing tensors, wrong shapes and bias tensors
(tools/convert_hf_llama.py:512-525).  Here the parts of the assembled model say
which tensors they bind (:class:`TensorRequest`); the loader compares that list
with what the checkpoint holds and raises one :class:`WeightError` naming every
missing tensor, every unexpected tensor and every wrong shape.

Storage policy.  ``role`` decides the dtype a tensor is held in:

* ``"matmul"`` and ``"embedding"``: the compute dtype (bfloat16 on the serving
  path, float32 on the true 32-bit path);
* ``"scale"`` (norm weights and other per-channel vectors): float32 in both
  modes.  Widening a stored bfloat16 vector is exact, and a vector stored in
  32-bit stays 32-bit;
* ``"table"``: integer tables, held as int32.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .safetensors_io import Checkpoint


class WeightError(RuntimeError):
    """The checkpoint does not hold exactly the tensors the model binds."""

    def __init__(self, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 other: Sequence[str] = ()) -> None:
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.other = list(other)
        lines = ["checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): "
                         + ", ".join(self.unexpected))
        for name, found, expected in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(found)}, expected {list(expected)}")
        for message in self.other:
            lines.append("  " + message)
        super().__init__("\n".join(lines))


@dataclasses.dataclass(frozen=True)
class TensorRequest:
    name: str
    shape: Tuple[int, ...]
    role: str = "matmul"            # matmul | embedding | scale | table
    fallback: Optional[str] = None  # another tensor that may stand in (tied weights)


_FLOAT_STORAGE = {"F32", "F16", "BF16"}
_INT_STORAGE = {"I32", "I64"}


def held_dtype(role: str, compute_dtype: torch.dtype) -> torch.dtype:
    if role in ("matmul", "embedding"):
        return compute_dtype
    if role == "scale":
        return torch.float32
    if role == "table":
        return torch.int32
    raise ValueError(f"unknown tensor role {role!r}")


def check_checkpoint(checkpoint: Checkpoint, requests: Iterable[TensorRequest]) -> Dict[str, str]:
    """Return ``request name -> source name`` or raise one WeightError for everything wrong."""
    available = set(checkpoint.names())
    missing: List[str] = []
    wrong: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]] = []
    other: List[str] = []
    used = set()
    sources: Dict[str, str] = {}
    for request in requests:
        source = request.name
        if source not in available:
            if request.fallback is not None and request.fallback in available:
                source = request.fallback
            else:
                missing.append(request.name)
                continue
        used.add(source)
        record = checkpoint.record(source)
        if tuple(record.shape) != tuple(request.shape):
            wrong.append((source, tuple(record.shape), tuple(request.shape)))
        allowed = _INT_STORAGE if request.role == "table" else _FLOAT_STORAGE
        if record.dtype not in allowed:
            other.append(f"wrong dtype: {source} is stored as {record.dtype}, "
                         f"expected one of {sorted(allowed)}")
        sources[request.name] = source
    unexpected = sorted(available - used)
    if missing or unexpected or wrong or other:
        raise WeightError(sorted(missing), unexpected, wrong, other)
    return sources


def load_tensors(checkpoint: Checkpoint, requests: Sequence[TensorRequest],
                 compute_dtype: torch.dtype, device: torch.device) -> Dict[str, torch.Tensor]:
    """Check, then read every requested tensor onto ``device`` in its held dtype."""
    sources = check_checkpoint(checkpoint, requests)
    result: Dict[str, torch.Tensor] = {}
    nonfinite: List[str] = []
    for request in requests:
        tensor = checkpoint.read(sources[request.name])
        if tensor.is_floating_point() and not bool(torch.isfinite(tensor.float()).all()):
            nonfinite.append(f"non-finite values in {sources[request.name]}")
            continue
        result[request.name] = tensor.to(device=device,
                                         dtype=held_dtype(request.role, compute_dtype))
    if nonfinite:
        raise WeightError((), (), (), nonfinite)
    return result
