"""The safetensors container: a reader over a memory map and a writer.

A file is an 8-byte little-endian header length, a JSON header that maps each tensor name to
``{dtype, shape, data_offsets}``, and one data buffer.  The reader turns the header into a
table of :class:`TensorRecord` and then checks the table as a whole: every record's byte
range must match its shape and dtype, and the ranges, sorted, must tile the data buffer
exactly (no overlap, no hole, nothing behind the last one).  Tensors are views into one
read-only memory map of the file, copied out when read.  The reference's converter applies
the same rules to the same format (tools/convert_hf_llama.py:208-313) and resolves sharded
checkpoints inside the folder only (tools/convert_hf_llama.py:316-368).
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Mapping, NamedTuple, Optional, Tuple

import numpy as np
import torch

from ..config.strict_json import parse_object

MAX_HEADER_BYTES = 100_000_000
INDEX_NAME = "model.safetensors.index.json"
SINGLE_NAME = "model.safetensors"


class SafetensorsError(RuntimeError):
    """The file is not a well-formed safetensors container."""


class _Storage(NamedTuple):
    numpy: str              # how numpy reads the stored bytes
    torch: torch.dtype
    bytes: int


STORAGE: Dict[str, _Storage] = {
    "F32": _Storage("<f4", torch.float32, 4),
    "F16": _Storage("<f2", torch.float16, 2),
    "BF16": _Storage("<i2", torch.bfloat16, 2),     # read as 16-bit integers, then reinterpreted
    "I32": _Storage("<i4", torch.int32, 4),
    "I64": _Storage("<i8", torch.int64, 8),
}
_NAME_OF = {storage.torch: name for name, storage in STORAGE.items()}


class TensorRecord(NamedTuple):
    name: str
    dtype: str
    shape: Tuple[int, ...]
    start: int
    end: int


def _is_count(value) -> bool:
    return isinstance(value, int) and not isinstance(value, bool) and value >= 0


def _record_from(where: str, name: str, entry, data_bytes: int) -> TensorRecord:
    """One header entry as a record, or a SafetensorsError that says what is wrong with it."""
    def bad(problem: str) -> SafetensorsError:
        return SafetensorsError(f"{where}: tensor {name!r} {problem}")

    if not isinstance(entry, dict) or sorted(entry) != ["data_offsets", "dtype", "shape"]:
        raise bad("has noncanonical metadata (exactly dtype, shape, data_offsets)")
    storage = STORAGE.get(entry["dtype"]) if isinstance(entry["dtype"], str) else None
    if storage is None:
        raise bad(f"uses unsupported dtype {entry['dtype']!r}")
    shape, offsets = entry["shape"], entry["data_offsets"]
    if not isinstance(shape, list) or not all(_is_count(extent) for extent in shape):
        raise bad("has an invalid shape")
    if not isinstance(offsets, list) or len(offsets) != 2 or not all(map(_is_count, offsets)):
        raise bad("has invalid data offsets")
    start, end = offsets
    if not start <= end <= data_bytes:
        raise bad("exceeds data-buffer bounds")
    if end - start != math.prod(shape) * storage.bytes:
        raise bad("has a byte range that does not match its shape and dtype")
    return TensorRecord(name, entry["dtype"], tuple(shape), start, end)


def _check_tiling(where: str, records: List[TensorRecord], data_bytes: int) -> None:
    """The byte ranges, in file order, must follow one another from 0 to the buffer's end."""
    ordered = sorted(records, key=lambda record: (record.start, record.end))
    expected = 0
    for record in ordered:
        if record.start < expected:
            raise SafetensorsError(f"{where}: tensor {record.name!r} overlaps a prior tensor")
        if record.start > expected:
            raise SafetensorsError(f"{where}: tensor {record.name!r} leaves a data hole")
        expected = record.end
    if expected != data_bytes:
        raise SafetensorsError(f"{where}: data buffer has trailing unclaimed bytes")


class SafetensorsFile:
    """One container file: its record table and a read-only map of its data buffer."""

    def __init__(self, path: str) -> None:
        self.path = path
        try:
            size = os.path.getsize(path)
            with open(path, "rb") as source:
                prefix = source.read(8)
                if len(prefix) < 8:
                    raise SafetensorsError(f"{path}: missing header length")
                (header_bytes,) = struct.unpack("<Q", prefix)
                if header_bytes > MAX_HEADER_BYTES:
                    raise SafetensorsError(f"{path}: header exceeds {MAX_HEADER_BYTES} bytes")
                if 8 + header_bytes > size:
                    raise SafetensorsError(f"{path}: header exceeds file bounds")
                text = source.read(header_bytes)
        except OSError as problem:
            raise SafetensorsError(f"could not read {path}: {problem}") from problem
        header = parse_object(text, f"{path}: header", SafetensorsError)
        self.data_offset = 8 + header_bytes
        data_bytes = size - self.data_offset
        self.records: Dict[str, TensorRecord] = {
            name: _record_from(path, name, entry, data_bytes)
            for name, entry in header.items() if name != "__metadata__"}
        _check_tiling(path, list(self.records.values()), data_bytes)
        self._map: Optional[np.memmap] = None

    def _data(self) -> np.ndarray:
        if self._map is None:
            self._map = np.memmap(self.path, dtype=np.uint8, mode="r", offset=self.data_offset) \
                if os.path.getsize(self.path) > self.data_offset else np.zeros(0, dtype=np.uint8)
        return self._map

    def read(self, name: str) -> torch.Tensor:
        """The tensor in its stored dtype: a fresh CPU tensor that owns its memory."""
        record = self.records[name]
        storage = STORAGE[record.dtype]
        raw = np.array(self._data()[record.start:record.end])          # copy out of the map
        tensor = torch.from_numpy(raw.view(storage.numpy).reshape(record.shape))
        return tensor.view(storage.torch) if record.dtype == "BF16" else tensor


class Checkpoint:
    """Every tensor of a model folder, whether it is one file or an index over shards."""

    def __init__(self, directory: str) -> None:
        self.directory = os.path.realpath(directory)
        if not os.path.isdir(self.directory):
            raise SafetensorsError(f"checkpoint path is not a directory: {directory}")
        self._files: Dict[str, SafetensorsFile] = {}
        self._home: Dict[str, SafetensorsFile] = {}
        for name, filename in self._placement().items():
            shard = self._shard(filename)
            if name not in shard.records:
                raise SafetensorsError(
                    f"index maps tensor {name!r} to {filename}, but the shard lacks it")
            self._home[name] = shard

    def _placement(self) -> Dict[str, Optional[str]]:
        """``tensor name -> shard file name`` from the index, or from the single file."""
        index_path = os.path.join(self.directory, INDEX_NAME)
        if os.path.exists(index_path):
            with open(index_path, "rb") as source:
                index = parse_object(source.read(), index_path, SafetensorsError)
            placement = index.get("weight_map")
            if not isinstance(placement, dict) or not all(
                    isinstance(filename, str) and filename for filename in placement.values()):
                raise SafetensorsError("index weight_map must map tensor names to files")
            return placement
        if os.path.exists(os.path.join(self.directory, SINGLE_NAME)):
            return {name: SINGLE_NAME for name in self._shard(SINGLE_NAME).records}
        raise SafetensorsError(f"{self.directory} contains neither {SINGLE_NAME} nor {INDEX_NAME}")

    def _shard(self, filename: str) -> SafetensorsFile:
        """The opened shard; a name that leads out of the folder is refused."""
        path = os.path.realpath(os.path.join(self.directory, filename))
        leaves = os.path.relpath(path, self.directory).split(os.sep)[0] == os.pardir
        if leaves or not os.path.isfile(path):
            raise SafetensorsError(
                f"index shard {filename!r} does not resolve inside the checkpoint")
        if path not in self._files:
            self._files[path] = SafetensorsFile(path)
        return self._files[path]

    def names(self) -> List[str]:
        return list(self._home)

    def record(self, name: str) -> TensorRecord:
        return self._home[name].records[name]

    def read(self, name: str) -> torch.Tensor:
        return self._home[name].read(name)


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                      metadata: Optional[Mapping[str, str]] = None) -> None:
    """Write ``tensors`` in insertion order, payloads back to back."""
    payloads: List[bytes] = []
    header: Dict[str, object] = {"__metadata__": dict(metadata)} if metadata else {}
    end = 0
    for name, tensor in tensors.items():
        stored = _NAME_OF.get(tensor.dtype)
        if stored is None:
            raise SafetensorsError(f"tensor {name!r} has unsupported dtype {tensor.dtype}")
        data = tensor.detach().contiguous().cpu()
        if stored == "BF16":
            data = data.view(torch.int16)
        payloads.append(data.numpy().astype(STORAGE[stored].numpy, copy=False).tobytes())
        header[name] = {"dtype": stored, "shape": list(tensor.shape),
                        "data_offsets": [end, end + len(payloads[-1])]}
        end += len(payloads[-1])
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)                 # the data buffer starts 8-byte aligned
    with open(path, "wb") as output:
        output.write(struct.pack("<Q", len(text)))
        output.write(text)
        for payload in payloads:
            output.write(payload)
