"""Helix's native model file: what the reader accepts, what it refuses, and the writer.

``tests/golden/tiny_A.helix`` was written by the reference's own converter and packer
(see ``tests/golden/make_golden.py``).  Every test that damages it changes ONE thing and,
where the damage sits in the header or the directory, seals the metadata checksum again, so
that the check under test is the one that fires (src/model/format.cpp:749-854, 1050-1079
are the reference's refusals).  The plain FNV-1a below is the test's own.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np
import pytest
import torch

from helix_runtime_b200.weights import (Checkpoint, HelixFile, HelixFileError, WeightError,
                                        check_checkpoint, open_model, write_helix_file)
from helix_runtime_b200.config import ConfigError
from tiny_configs import make_folder, tiny_config

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tiny_A.helix")
HEADER, ENTRY = 128, 80


def plain_fnv1a(data: bytes) -> int:
    value = 14695981039346656037
    for byte in data:
        value = ((value ^ byte) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return value


def golden_bytes() -> bytearray:
    with open(GOLDEN, "rb") as source:
        return bytearray(source.read())


def sealed(data: bytearray) -> bytearray:
    """Recompute the metadata checksum over the (changed) header and directory."""
    count = struct.unpack_from("<Q", data, 40)[0]
    end = HEADER + ENTRY * min(count, 64)
    data[120:128] = bytes(8)
    data[120:128] = struct.pack("<Q", plain_fnv1a(bytes(data[:end])))
    return data


def refused(tmp_path, data: bytes, match: str) -> None:
    path = tmp_path / "damaged.helix"
    path.write_bytes(bytes(data))
    with pytest.raises(HelixFileError, match=match):
        HelixFile(str(path))


def test_reads_the_reference_made_file_as_the_folder_it_was_converted_from(model_root):
    source = HelixFile(GOLDEN)
    document = source.config_document()
    expected = tiny_config("A").to_dict()
    for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                "num_attention_heads", "num_key_value_heads", "head_dim",
                "max_position_embeddings", "model_type"):
        assert document[key] == expected[key], key
    assert document["rms_norm_eps"] == float(np.float32(expected["rms_norm_eps"]))
    folder = make_folder(model_root, "A", storage_dtype="float32")
    checkpoint = Checkpoint(folder)
    assert sorted(source.names()) == sorted(checkpoint.names())
    same = all(torch.equal(source.read(name), checkpoint.read(name).float())
               for name in checkpoint.names())
    if not same:
        pytest.skip("this torch build draws other random weights than the one that made the "
                    "golden files; rerun tests/golden/make_golden.py")
    # the metadata checksum in the file is the plain FNV-1a of header (field zeroed) + directory
    data = golden_bytes()
    stored = struct.unpack_from("<Q", data, 120)[0]
    assert struct.unpack_from("<Q", sealed(data), 120)[0] == stored


def test_the_writer_reproduces_the_reference_made_file_byte_for_byte(model_root, tmp_path):
    folder = make_folder(model_root, "A", storage_dtype="float32")
    checkpoint = Checkpoint(folder)
    with open(os.path.join(folder, "config.json")) as source:
        document = json.load(source)
    path = str(tmp_path / "again.helix")
    write_helix_file(path, document, {name: checkpoint.read(name) for name in checkpoint.names()})
    with open(path, "rb") as source:
        written = source.read()
    if len(written) == len(golden_bytes()) and written != bytes(golden_bytes()):
        same_weights = all(torch.equal(HelixFile(GOLDEN).read(n), checkpoint.read(n).float())
                           for n in checkpoint.names())
        if not same_weights:
            pytest.skip("other random weights than the golden file's")
    assert written == bytes(golden_bytes())


def test_another_configuration_round_trips_through_the_file(model_root, tmp_path):
    folder = make_folder(model_root, "B", storage_dtype="bfloat16")
    document, checkpoint = open_model(folder)
    path = str(tmp_path / "tiny_B.helix")
    write_helix_file(path, document, {name: checkpoint.read(name) for name in checkpoint.names()})
    document_again, source = open_model(path)
    assert document_again["num_hidden_layers"] == 3 and document_again["head_dim"] == 24
    assert document_again["rope_theta"] == 500000.0
    for name in checkpoint.names():
        record = source.record(name)
        assert record.dtype == "F32" and record.shape == checkpoint.record(name).shape
        assert torch.equal(source.read(name), checkpoint.read(name).float()), name
    # the loader's one error also speaks about a file: a model with one layer more
    from helix_runtime_b200 import LlamaConfig
    from helix_runtime_b200.models.decoder import DecoderModel
    from helix_runtime_b200.config import architecture_for
    larger = dict(document_again, num_hidden_layers=4)
    architecture = architecture_for(larger)
    model = DecoderModel(architecture.build_spec(LlamaConfig.from_dict(larger)))
    with pytest.raises(WeightError, match="missing tensors"):
        check_checkpoint(source, model.tensor_requests())


def test_header_damage_is_refused_field_by_field(tmp_path):
    cases = [
        (0, b"X", "magic"),                                   # magic
        (8, struct.pack("<I", 2), "format version"),          # version
        (12, struct.pack("<I", 0x04030201), "endianness"),    # big-endian marker
        (16, struct.pack("<I", 256), "header size"),
        (20, struct.pack("<I", 7), "model kind"),
        (24, struct.pack("<Q", 535617), "declares 535617 bytes"),   # declared size
        (32, struct.pack("<Q", 192), "directory does not start"),
        (40, struct.pack("<Q", 20), "20 tensors in the directory"),
        (48, struct.pack("<Q", 96), "entry size"),
        (56, struct.pack("<Q", 1920), "data offset"),
        (64, struct.pack("<Q", 0), "vocabulary size"),
        (96, struct.pack("<Q", 3), "does not split into 3"),        # heads
        (112, struct.pack("<f", float("nan")), "positive and finite"),
    ]
    for offset, patch, message in cases:
        data = golden_bytes()
        data[offset:offset + len(patch)] = patch
        refused(tmp_path, sealed(data), message)
    # one byte of the header changed and NOT sealed: the metadata checksum catches it
    data = golden_bytes()
    data[113] ^= 0x01
    refused(tmp_path, data, "metadata checksum mismatch")
    # the checksum field itself
    data = golden_bytes()
    data[121] ^= 0x40
    refused(tmp_path, data, "metadata checksum mismatch")


def test_directory_damage_is_refused(tmp_path):
    first, second = HEADER, HEADER + ENTRY
    cases = [
        (first, struct.pack("<I", 2), "should be token_embedding"),          # role
        (second + 4, struct.pack("<I", 1), "should be attention_norm of layer 0"),
        (second + 8, struct.pack("<I", 2), "dtype code"),
        (second + 12, struct.pack("<I", 2), "rank 2, expected 1"),
        (first + 16, struct.pack("<Q", 255), "unexpected shape"),
        (first + 56, struct.pack("<Q", 65540), "invalid byte length"),
        (first + 48, struct.pack("<Q", 1920), "non-canonical payload offset"),
        (first + 64, struct.pack("<Q", 128), "non-canonical payload offset"),   # alignment
    ]
    for offset, patch, message in cases:
        data = golden_bytes()
        data[offset:offset + len(patch)] = patch
        refused(tmp_path, sealed(data), message)
    data = golden_bytes()
    data[first + 17] ^= 0x01                      # unsealed directory byte
    refused(tmp_path, data, "metadata checksum mismatch")


def test_payload_padding_size_and_trailing_bytes(tmp_path):
    data = golden_bytes()
    data_offset = struct.unpack_from("<Q", data, 56)[0]
    # a payload value changed: the tensor's own checksum
    data[data_offset + 5] ^= 0x10
    refused(tmp_path, data, "token_embedding: payload checksum mismatch")
    # a stored checksum changed (sealed, so the metadata agrees with itself)
    data = golden_bytes()
    data[HEADER + 72] ^= 0x01
    refused(tmp_path, sealed(data), "token_embedding: payload checksum mismatch")
    # a non-finite value whose checksum is right
    data = golden_bytes()
    entry = HEADER + ENTRY * 2                    # query projection of layer 0
    offset, length = struct.unpack_from("<QQ", data, entry + 48)
    data[offset + 8:offset + 12] = struct.pack("<f", float("inf"))
    data[entry + 72:entry + 80] = struct.pack("<Q", plain_fnv1a(bytes(data[offset:offset + length])))
    refused(tmp_path, sealed(data), "query of layer 0 contains a non-finite value")
    # padding: between the directory's end (128 + 21 * 80 = 1808) and the first payload (1856)
    data = golden_bytes()
    assert data_offset == 1856 and not any(data[1808:1856])
    data[1830] = 1
    refused(tmp_path, data, "padding before token_embedding")
    # trailing bytes, declared or not
    data = golden_bytes() + bytearray(64)
    refused(tmp_path, data, "declares 535616 bytes, the file has 535680")
    data[24:32] = struct.pack("<Q", len(data))
    refused(tmp_path, sealed(data), "64 trailing bytes")
    # cut short
    data = golden_bytes()[:-4]
    refused(tmp_path, data, "declares")
    data[24:32] = struct.pack("<Q", len(data))
    refused(tmp_path, sealed(data), "payloads need 535616 bytes")
    refused(tmp_path, golden_bytes()[:100], "smaller than the 128-byte header")


def test_what_is_neither_a_folder_nor_a_model_file(tmp_path):
    with pytest.raises(ConfigError, match="neither a model folder"):
        open_model(str(tmp_path / "nothing_here"))
    other = tmp_path / "notes.helix"
    other.write_bytes(b"these are not the bytes of a model file, " * 8)
    with pytest.raises(HelixFileError, match="magic"):
        open_model(str(other))
