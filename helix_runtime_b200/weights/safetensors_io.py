"""A small reader and writer for the safetensors container.

Format: 8-byte little-endian header length, a JSON header mapping each tensor
name to ``{dtype, shape, data_offsets}``, then the raw little-endian payloads.
The checks mirror the reference's own parser (tools/convert_hf_llama.py:208-313):
bounded header, canonical record fields, byte range equal to shape × dtype size,
payloads that neither overlap nor leave holes, no trailing bytes.  Sharded
checkpoints (``model.safetensors.index.json``) are resolved inside the folder
only (tools/convert_hf_llama.py:357-368).
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, Iterable, List, Mapping, NamedTuple, Optional, Tuple

import numpy as np
import torch

MAX_HEADER_BYTES = 100_000_000

_DTYPE_BYTES = {"F32": 4, "F16": 2, "BF16": 2, "I32": 4, "I64": 8}
_NUMPY_DTYPE = {"F32": "<f4", "F16": "<f2", "BF16": "<u2", "I32": "<i4", "I64": "<i8"}
_TORCH_TO_NAME = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
                  torch.int32: "I32", torch.int64: "I64"}


class SafetensorsError(RuntimeError):
    """The file is not a well-formed safetensors container."""


class TensorRecord(NamedTuple):
    name: str
    dtype: str
    shape: Tuple[int, ...]
    start: int
    end: int


def _strict_object(pairs):
    result = {}
    for key, value in pairs:
        if key in result:
            raise SafetensorsError(f"JSON object contains duplicate key {key!r}")
        result[key] = value
    return result


class SafetensorsFile:
    """Header of one file plus lazy, memory-mapped access to its tensors."""

    def __init__(self, path: str) -> None:
        self.path = path
        try:
            file_size = os.stat(path).st_size
            with open(path, "rb") as source:
                length_bytes = source.read(8)
                if len(length_bytes) != 8:
                    raise SafetensorsError(f"{path}: missing header length")
                (header_length,) = struct.unpack("<Q", length_bytes)
                if header_length > MAX_HEADER_BYTES:
                    raise SafetensorsError(f"{path}: header exceeds {MAX_HEADER_BYTES} bytes")
                if header_length > file_size - 8:
                    raise SafetensorsError(f"{path}: header exceeds file bounds")
                header_bytes = source.read(header_length)
        except OSError as error:
            raise SafetensorsError(f"could not read {path}: {error}") from error
        try:
            header = json.loads(header_bytes.decode("utf-8"), object_pairs_hook=_strict_object)
        except (UnicodeError, json.JSONDecodeError) as error:
            raise SafetensorsError(f"{path}: invalid JSON header: {error}") from error
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be an object")
        header.pop("__metadata__", None)

        data_bytes = file_size - 8 - header_length
        self.data_offset = 8 + header_length
        self.records: Dict[str, TensorRecord] = {}
        ranges: List[Tuple[int, int, str]] = []
        for name, record in header.items():
            if not isinstance(record, dict) or set(record) != {"dtype", "shape", "data_offsets"}:
                raise SafetensorsError(f"{path}: tensor {name!r} has noncanonical metadata")
            dtype = record["dtype"]
            if dtype not in _DTYPE_BYTES:
                raise SafetensorsError(f"{path}: tensor {name!r} uses unsupported dtype {dtype!r}")
            shape = record["shape"]
            if not isinstance(shape, list) or any(
                    isinstance(d, bool) or not isinstance(d, int) or d < 0 for d in shape):
                raise SafetensorsError(f"{path}: tensor {name!r} has an invalid shape")
            offsets = record["data_offsets"]
            if (not isinstance(offsets, list) or len(offsets) != 2 or any(
                    isinstance(o, bool) or not isinstance(o, int) for o in offsets)):
                raise SafetensorsError(f"{path}: tensor {name!r} has invalid data offsets")
            start, end = offsets
            if start < 0 or end < start or end > data_bytes:
                raise SafetensorsError(f"{path}: tensor {name!r} exceeds data-buffer bounds")
            if end - start != math.prod(shape) * _DTYPE_BYTES[dtype]:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} byte range does not match its shape/dtype")
            self.records[name] = TensorRecord(name, dtype, tuple(shape), start, end)
            ranges.append((start, end, name))
        cursor = 0
        for start, end, name in sorted(ranges):
            if start != cursor:
                relation = "overlaps a prior tensor" if start < cursor else "leaves a data hole"
                raise SafetensorsError(f"{path}: tensor {name!r} {relation}")
            cursor = end
        if cursor != data_bytes:
            raise SafetensorsError(f"{path}: data buffer has trailing unclaimed bytes")

    def read(self, name: str) -> torch.Tensor:
        """Return the tensor in its stored dtype (a fresh CPU tensor)."""
        record = self.records[name]
        count = math.prod(record.shape)
        if count == 0:
            array = np.zeros(record.shape, dtype=np.dtype(_NUMPY_DTYPE[record.dtype]))
        else:
            array = np.fromfile(self.path, dtype=np.dtype(_NUMPY_DTYPE[record.dtype]),
                                count=count, offset=self.data_offset + record.start)
            array = array.reshape(record.shape)
        if record.dtype == "BF16":
            return torch.from_numpy(array.view(np.int16)).view(torch.bfloat16)
        return torch.from_numpy(array)


class Checkpoint:
    """All tensors of a model folder: one ``model.safetensors`` or an index of shards."""

    def __init__(self, directory: str) -> None:
        self.directory = os.path.realpath(directory)
        if not os.path.isdir(self.directory):
            raise SafetensorsError(f"checkpoint path is not a directory: {directory}")
        index_path = os.path.join(self.directory, "model.safetensors.index.json")
        single_path = os.path.join(self.directory, "model.safetensors")
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        if os.path.exists(index_path):
            with open(index_path, "r", encoding="utf-8") as source:
                index = json.load(source, object_pairs_hook=_strict_object)
            weight_map = index.get("weight_map") if isinstance(index, dict) else None
            if not isinstance(weight_map, dict) or any(
                    not isinstance(k, str) or not isinstance(v, str) or not v
                    for k, v in weight_map.items()):
                raise SafetensorsError("index weight_map must map tensor names to files")
            for name, filename in weight_map.items():
                resolved = os.path.realpath(os.path.join(self.directory, filename))
                if os.path.commonpath([resolved, self.directory]) != self.directory \
                        or not os.path.isfile(resolved):
                    raise SafetensorsError(
                        f"index shard {filename!r} does not resolve inside the checkpoint")
                if resolved not in self._files:
                    self._files[resolved] = SafetensorsFile(resolved)
                if name not in self._files[resolved].records:
                    raise SafetensorsError(
                        f"index maps tensor {name!r} to {filename}, but the shard lacks it")
                self._where[name] = resolved
        elif os.path.exists(single_path):
            self._files[single_path] = SafetensorsFile(single_path)
            for name in self._files[single_path].records:
                self._where[name] = single_path
        else:
            raise SafetensorsError(
                f"{self.directory} contains neither model.safetensors nor "
                "model.safetensors.index.json")

    def names(self) -> List[str]:
        return list(self._where)

    def record(self, name: str) -> TensorRecord:
        return self._files[self._where[name]].records[name]

    def read(self, name: str) -> torch.Tensor:
        return self._files[self._where[name]].read(name)


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                      metadata: Optional[Mapping[str, str]] = None) -> None:
    """Write ``tensors`` (CPU, contiguous) in insertion order."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    cursor = 0
    for name, tensor in tensors.items():
        if tensor.dtype not in _TORCH_TO_NAME:
            raise SafetensorsError(f"tensor {name!r} has unsupported dtype {tensor.dtype}")
        size = tensor.numel() * tensor.element_size()
        header[name] = {"dtype": _TORCH_TO_NAME[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [cursor, cursor + size]}
        cursor += size
    header_bytes = json.dumps(header, separators=(",", ":")).encode("utf-8")
    header_bytes += b" " * ((8 - len(header_bytes) % 8) % 8)
    with open(path, "wb") as output:
        output.write(struct.pack("<Q", len(header_bytes)))
        output.write(header_bytes)
        for tensor in tensors.values():
            data = tensor.detach().contiguous().cpu()
            if data.dtype == torch.bfloat16:
                data = data.view(torch.int16)
            output.write(data.numpy().tobytes())


def iter_names(files: Iterable[SafetensorsFile]) -> Iterable[str]:
    for file in files:
        yield from file.records
