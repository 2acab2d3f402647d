"""The plain implementation against the reference's own compiled CPU model.

``tests/golden/make_golden.py`` ran the reference's converter and ``helix_model_inspect`` on
the two tiny model folders and stored its logits and greedy tokens; here the plain
implementation recomputes them.  Also: the plain model from the checkpoint's own layout
(half-split rotation) must equal the plain model in the reference's layout (adjacent pairs
after the row permutation).
"""
from __future__ import annotations

import hashlib
import json
import os

import numpy as np
import pytest

import plain_llama
from tiny_configs import make_folder

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_equals_reference_cpu_model(name, model_root):
    with open(os.path.join(GOLDEN, f"tiny_{name}.json"), "r", encoding="utf-8") as source:
        golden = json.load(source)
    folder = make_folder(model_root, name, storage_dtype="float32")
    with open(os.path.join(folder, "model.safetensors"), "rb") as source:
        checksum = hashlib.sha256(source.read()).hexdigest()
    if checksum != golden["weights_sha256"]:
        pytest.skip("this torch build draws other random weights than the one that made the "
                    "golden files; rerun tests/golden/make_golden.py")
    model = plain_llama.PlainModel(folder)
    tokens = golden["tokens"]
    for length, values in golden["last_logits_hex"].items():
        reference = np.asarray([float.fromhex(v) for v in values], dtype=np.float32)
        mine = model.logits(tokens[:int(length)])[-1]
        np.testing.assert_allclose(mine, reference, rtol=0, atol=5e-7,
                                   err_msg=f"tiny {name}, prefix of {length}")
    greedy = golden["greedy"]
    assert model.greedy(tokens[:greedy["prompt_length"]], len(greedy["tokens"])) == greedy["tokens"]


@pytest.mark.parametrize("name", ["A", "B"])
def test_checkpoint_layout_and_reference_layout_agree(name, model_root):
    folder = make_folder(model_root, name, storage_dtype="float32", sharp=True)
    model = plain_llama.PlainModel(folder)
    rng = np.random.default_rng(3)
    tokens = [int(t) for t in rng.integers(0, model.config["vocab_size"], size=23)]
    adjacent = model.logits(tokens)
    half_split = plain_llama.forward_source_layout(model.config, model.source, tokens)
    np.testing.assert_allclose(adjacent, half_split, rtol=0, atol=2e-6)


def test_parts_of_the_plain_implementation():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(3, 8)).astype(np.float32)
    w = rng.normal(size=8).astype(np.float32)
    expected = x / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-5) * w
    np.testing.assert_allclose(plain_llama.rms_norm(x, w, 1e-5), expected, rtol=1e-6)
    # silu at the branch point and far from it
    np.testing.assert_allclose(plain_llama.silu(np.array([0.0, 30.0, -30.0], dtype=np.float32)),
                               [0.0, 30.0, -30.0 * np.exp(-30.0)], rtol=1e-6, atol=1e-12)
    # rotation keeps pair norms and is the identity at position 0
    cosine, sine = plain_llama.rope_table(4, 8, 10000.0)
    q = rng.normal(size=(4, 2, 8)).astype(np.float32)
    rotated = plain_llama.rope_adjacent(q, cosine, sine)
    np.testing.assert_allclose(rotated[0], q[0], atol=1e-7)
    np.testing.assert_allclose(rotated[..., 0::2] ** 2 + rotated[..., 1::2] ** 2,
                               q[..., 0::2] ** 2 + q[..., 1::2] ** 2, rtol=1e-5)
    # causal: the first query sees only the first key
    k = rng.normal(size=(2, 4, 8)).astype(np.float32)
    v = rng.normal(size=(2, 4, 8)).astype(np.float32)
    out = plain_llama.causal_attention(q.transpose(1, 0, 2), k, v)
    np.testing.assert_allclose(out[:, 0], v[:, 0], atol=1e-6)
    # a window of one sees only the key at the query's own position
    out = plain_llama.causal_attention(q.transpose(1, 0, 2), k, v, window=1)
    np.testing.assert_allclose(out, v, atol=1e-6)
    # greedy takes the lowest id among equals and refuses non-finite rows
    assert plain_llama.select_greedy_token(np.array([1.0, 3.0, 3.0], dtype=np.float32)) == 1
    with pytest.raises(FloatingPointError):
        plain_llama.select_greedy_token(np.array([1.0, np.nan], dtype=np.float32))
