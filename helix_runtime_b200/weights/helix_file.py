"""Helix's native model file (``MODEL.helix``, magic ``HELIXLM1``) as a weight source.

The reference's own tools load this container (src/model/format.cpp:1050-1079): a 128-byte
header with the model's sizes, a directory of 80-byte entries, float32 payloads on 64-byte
boundaries, FNV-1a checksums of the metadata and of every payload.  Reading, and every
refusal (magic, version, endianness, sizes, directory order, shapes, offsets, padding,
checksums, non-finite values, trailing bytes), is done by the host library
(``csrc/host/hx_model_file.cpp``); this module is its Python face.

A :class:`HelixFile` looks like a checkpoint folder to the loader: it gives a
``config.json``-style document and tensors under the checkpoint names of
``tools/convert_hf_llama.py:400-510``, in that layout: ``[out, in]`` matrices (the file holds
``[in, out]``), and the rows of the query and key projections ordered for half-split rotation
(the file holds them ordered for adjacent pairs, tools/convert_hf_llama.py:535-542; the
inverse permutation is applied here).  So a model loaded from the file is bit for bit the
model loaded from the folder it was converted from.

:func:`write_helix_file` is the inverse: a folder's tensors written as the reference's
converter and packer write them.
"""
from __future__ import annotations

import ctypes
import os
import struct
import threading
from typing import Any, Dict, List, Mapping, Optional, Tuple

import numpy as np
import torch

from ..csrc import build as _build
from .safetensors_io import TensorRecord

MAGIC = b"HELIXLM1"
MODEL_KINDS = {1: ("llama", "LlamaForCausalLM")}     # src/model/format.cpp:44

_ROLE_NAMES = {
    1: "model.embed_tokens.weight",
    2: "model.layers.{layer}.input_layernorm.weight",
    3: "model.layers.{layer}.self_attn.q_proj.weight",
    4: "model.layers.{layer}.self_attn.k_proj.weight",
    5: "model.layers.{layer}.self_attn.v_proj.weight",
    6: "model.layers.{layer}.self_attn.o_proj.weight",
    7: "model.layers.{layer}.post_attention_layernorm.weight",
    8: "model.layers.{layer}.mlp.gate_proj.weight",
    9: "model.layers.{layer}.mlp.up_proj.weight",
    10: "model.layers.{layer}.mlp.down_proj.weight",
    11: "model.norm.weight",
    12: "lm_head.weight",
}
_ROTARY_ROLES = (3, 4)
# projections are held [in, out]; the embedding table keeps the checkpoint's [vocab, hidden]
_TRANSPOSED_ROLES = (3, 4, 5, 6, 8, 9, 10, 12)
_PER_LAYER_ROLES = tuple(range(2, 11))


class HelixFileError(RuntimeError):
    """The file is not a well-formed Helix model file, or could not be read."""


class _Config(ctypes.Structure):
    _fields_ = [("vocab_size", ctypes.c_uint64), ("hidden_size", ctypes.c_uint64),
                ("intermediate_size", ctypes.c_uint64), ("num_layers", ctypes.c_uint64),
                ("num_heads", ctypes.c_uint64), ("max_positions", ctypes.c_uint64),
                ("rms_norm_eps", ctypes.c_float), ("rope_theta", ctypes.c_float),
                ("model_kind", ctypes.c_uint32)]


class _Tensor(ctypes.Structure):
    _fields_ = [("role", ctypes.c_int), ("layer", ctypes.c_int), ("rank", ctypes.c_int),
                ("dims", ctypes.c_uint64 * 4), ("offset", ctypes.c_uint64),
                ("bytes", ctypes.c_uint64), ("checksum", ctypes.c_uint64),
                ("data", ctypes.c_void_p)]


_lock = threading.Lock()
_library: Optional[ctypes.CDLL] = None


def host_library() -> ctypes.CDLL:
    """The host library (compiled at first use with the C++ compiler; needs no GPU)."""
    global _library
    if _library is None:
        with _lock:
            if _library is None:
                library = ctypes.CDLL(_build.build_host())
                library.hx_host_last_error.restype = ctypes.c_char_p
                library.hx_fnv1a64.restype = ctypes.c_uint64
                library.hx_fnv1a64.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64]
                library.hx_model_file_open.argtypes = [ctypes.c_char_p,
                                                       ctypes.POINTER(ctypes.c_void_p)]
                library.hx_model_file_close.argtypes = [ctypes.c_void_p]
                library.hx_model_file_close.restype = None
                library.hx_model_file_config.argtypes = [ctypes.c_void_p, ctypes.POINTER(_Config)]
                library.hx_model_file_tensor_count.argtypes = [ctypes.c_void_p]
                library.hx_model_file_tensor_count.restype = ctypes.c_longlong
                library.hx_model_file_tensor.argtypes = [ctypes.c_void_p, ctypes.c_longlong,
                                                         ctypes.POINTER(_Tensor)]
                library.hx_model_file_verify.argtypes = [ctypes.c_void_p, ctypes.c_int]
                _library = library
    return _library


def fnv1a64(data: bytes, seed: int = 0) -> int:
    """FNV-1a (64-bit) of ``data``, continuing from ``seed`` (0: the standard basis)."""
    return int(host_library().hx_fnv1a64(data, len(data), seed))


def is_helix_file(path: str) -> bool:
    """A regular file that starts with the container's magic bytes."""
    if not os.path.isfile(path):
        return False
    try:
        with open(path, "rb") as source:
            return source.read(len(MAGIC)) == MAGIC
    except OSError:
        return False


def _half_split_rows(heads: int, head_dim: int) -> np.ndarray:
    """For a matrix whose rows are ordered for adjacent-pair rotation, the row order that
    restores the checkpoint's half-split order: new row ``f`` is old row ``2f``, new row
    ``D/2 + f`` is old row ``2f + 1``, head by head."""
    within = np.concatenate([np.arange(0, head_dim, 2), np.arange(1, head_dim, 2)])
    return (np.arange(heads)[:, None] * head_dim + within[None, :]).reshape(-1)


def _adjacent_rows(heads: int, head_dim: int) -> np.ndarray:
    """The inverse: from half-split order to adjacent pairs (tools/convert_hf_llama.py:535-542)."""
    order = np.empty(heads * head_dim, dtype=np.int64)
    order[_half_split_rows(heads, head_dim)] = np.arange(heads * head_dim)
    return order


class HelixFile:
    """An opened, checked model file; a weight source with a checkpoint's interface."""

    def __init__(self, path: str, verify: bool = True, threads: Optional[int] = None) -> None:
        self.path = path
        library = host_library()
        handle = ctypes.c_void_p()
        if library.hx_model_file_open(os.fsencode(path), ctypes.byref(handle)) != 0:
            raise HelixFileError(library.hx_host_last_error().decode("utf-8", "replace"))
        self._handle = handle
        self._library = library
        try:
            if verify and library.hx_model_file_verify(
                    handle, threads or min(8, os.cpu_count() or 1)) != 0:
                raise HelixFileError(f"{path}: " +
                                     library.hx_host_last_error().decode("utf-8", "replace"))
            config = _Config()
            library.hx_model_file_config(handle, ctypes.byref(config))
            self.config = config
            self.head_dim = int(config.hidden_size // config.num_heads)
            self._tensors: Dict[str, _Tensor] = {}
            for index in range(library.hx_model_file_tensor_count(handle)):
                tensor = _Tensor()
                library.hx_model_file_tensor(handle, index, ctypes.byref(tensor))
                self._tensors[_ROLE_NAMES[tensor.role].format(layer=tensor.layer)] = tensor
        except Exception:
            self.close()
            raise

    def close(self) -> None:
        if self._handle is not None:
            self._library.hx_model_file_close(self._handle)
            self._handle = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------- configuration

    def config_document(self) -> Dict[str, Any]:
        """The sizes of the header as the ``config.json`` the converter would have read.
        Epsilon and the rotary base are the file's float32 values."""
        c = self.config
        model_type, architecture = MODEL_KINDS[int(c.model_kind)]
        return {
            "architectures": [architecture], "model_type": model_type,
            "vocab_size": int(c.vocab_size), "hidden_size": int(c.hidden_size),
            "intermediate_size": int(c.intermediate_size),
            "num_hidden_layers": int(c.num_layers), "num_attention_heads": int(c.num_heads),
            "num_key_value_heads": int(c.num_heads), "head_dim": self.head_dim,
            "max_position_embeddings": int(c.max_positions), "hidden_act": "silu",
            "rms_norm_eps": float(c.rms_norm_eps), "rope_theta": float(c.rope_theta),
            "rope_scaling": None, "attention_bias": False, "mlp_bias": False,
            "tie_word_embeddings": False,
        }

    # ------------------------------------------------------- checkpoint interface

    def names(self) -> List[str]:
        return list(self._tensors)

    def record(self, name: str) -> TensorRecord:
        tensor = self._tensors[name]
        shape = tuple(int(d) for d in tensor.dims[:tensor.rank])
        if tensor.role in _TRANSPOSED_ROLES:
            shape = (shape[1], shape[0])          # the file holds [in, out]
        return TensorRecord(name, "F32", shape, int(tensor.offset),
                            int(tensor.offset + tensor.bytes))

    def stored(self, name: str) -> np.ndarray:
        """The payload as the file holds it (a read-only view of the mapping)."""
        tensor = self._tensors[name]
        shape = tuple(int(d) for d in tensor.dims[:tensor.rank])
        buffer = (ctypes.c_char * int(tensor.bytes)).from_address(tensor.data)
        array = np.frombuffer(buffer, dtype="<f4").reshape(shape)
        array.flags.writeable = False
        return array

    def read(self, name: str) -> torch.Tensor:
        """The tensor in the checkpoint's layout (a fresh CPU tensor, float32)."""
        tensor = self._tensors[name]
        array = self.stored(name)
        if tensor.role in _TRANSPOSED_ROLES:
            array = array.T
            if tensor.role in _ROTARY_ROLES:
                array = array[_half_split_rows(int(self.config.num_heads), self.head_dim)]
        return torch.from_numpy(np.array(array, dtype=np.float32, order="C"))   # a copy


# ---------------------------------------------------------------------- writing

def write_helix_file(path: str, document: Mapping[str, Any],
                     tensors: Mapping[str, torch.Tensor]) -> None:
    """Write ``tensors`` (checkpoint names and layout) as a Helix model file: float32,
    ``[in, out]`` matrices, query and key rows ordered for adjacent-pair rotation, and the
    layout and checksums of src/model/format.cpp:474-550."""
    heads = int(document["num_attention_heads"])
    hidden = int(document["hidden_size"])
    layers = int(document["num_hidden_layers"])
    if int(document.get("num_key_value_heads", heads) or heads) != heads:
        raise HelixFileError("the container holds equal query and key/value heads only")
    head_dim = hidden // heads
    tied = bool(document.get("tie_word_embeddings", False))

    def payload(role: int, layer: int) -> Tuple[np.ndarray, Tuple[int, ...]]:
        name = _ROLE_NAMES[role].format(layer=layer)
        if name not in tensors and role == 12 and tied:
            name = _ROLE_NAMES[1]
        if name not in tensors:
            raise HelixFileError(f"tensor {name!r} is missing")
        array = tensors[name].detach().to(torch.float32).cpu().numpy()
        if role in _TRANSPOSED_ROLES:
            if role in _ROTARY_ROLES:
                array = array[_adjacent_rows(heads, head_dim)]
            array = array.T
        array = np.ascontiguousarray(array, dtype="<f4")
        if not np.isfinite(array).all():
            raise HelixFileError(f"tensor {name!r} contains a non-finite value")
        return array, array.shape

    order = [(1, -1)] + [(role, layer) for layer in range(layers) for role in _PER_LAYER_ROLES] \
        + [(11, -1), (12, -1)]
    directory_end = 128 + 80 * len(order)
    data_offset = -(-directory_end // 64) * 64
    library = host_library()
    entries: List[bytes] = []
    cursor = data_offset
    partial = f"{path}.{os.getpid()}.tmp"
    with open(partial, "wb") as output:
        output.write(b"\0" * data_offset)          # header and directory follow at the end
        for role, layer in order:
            array, shape = payload(role, layer)
            aligned = -(-cursor // 64) * 64
            output.write(b"\0" * (aligned - cursor))
            data = array.tobytes()
            output.write(data)
            dims = list(shape) + [0] * (4 - len(shape))
            entries.append(struct.pack("<IIII4QQQQQ", role, layer & 0xFFFFFFFF, 1, len(shape),
                                       *dims, aligned, len(data), 64,
                                       library.hx_fnv1a64(data, len(data), 0)))
            cursor = aligned + len(data)
        directory = b"".join(entries)
        eps = float(np.float32(document.get("rms_norm_eps", 1.0e-6)))
        theta = float(np.float32(document.get("rope_theta", 10000.0)))
        header = MAGIC + struct.pack(
            "<IIIIQQQQQQQQQQQffQ", 1, 0x01020304, 128, 1, cursor, 128, len(order), 80, data_offset,
            int(document["vocab_size"]), hidden, int(document["intermediate_size"]), layers, heads,
            int(document["max_position_embeddings"]), eps, theta, 0)
        checksum = fnv1a64(header + directory)
        output.seek(0)
        output.write(header[:-8] + struct.pack("<Q", checksum) + directory)
    os.replace(partial, path)
