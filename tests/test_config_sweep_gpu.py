"""Further shapes of the architecture through the whole engine against the plain
implementation: head sizes from 6 to 256 (every kernel family of the attention: general,
16-byte pieces, tensor cores), widths that are no multiple of 8 (bfloat16 products then run on
the CUDA-core kernel), odd vocabularies, pages of 2 to 128 keys.  Each shape runs whole
requests and mixed batches over a pool so small that pages are used again, in float32 and in
bfloat16.

The bfloat16 bound is not a constant: rounding to bfloat16 moves the logits of a model by an
amount that grows with its width, and that amount is measured here with the plain
implementation itself (float32 against the same model with activations rounded where a
bfloat16 engine stores them).  The engine must stay within 0.8 of it, the same factor the
fixed tolerances of the tiny configurations stand for; a wrong key, page or tile moves a
logit by several times that amount.
"""
from __future__ import annotations

import os

import numpy as np
import pytest

import plain_llama
import traces
from conftest import random_tokens
from engine_harness import BF16_TOL, F32_TOL, Harness, assert_close
from helix_runtime_b200 import LlamaConfig, write_random_model
from tiny_configs import SCORE_SPREAD

pytestmark = pytest.mark.gpu

# heads, head size, intermediate, vocabulary, layers, page size
SHAPES = [
    (7, 6, 50, 131, 2, 4),
    (5, 10, 36, 99, 2, 8),
    (9, 16, 100, 201, 1, 2),
    (3, 32, 200, 300, 2, 8),
    (2, 48, 136, 260, 2, 16),
    (3, 80, 392, 333, 1, 16),
    (2, 96, 264, 515, 2, 64),
    (1, 112, 128, 257, 2, 16),
    (3, 128, 640, 777, 2, 16),
    (4, 64, 384, 512, 2, 128),
    (2, 192, 200, 300, 1, 8),
    (2, 256, 512, 400, 1, 16),
]
LENGTHS = (3, 40, 130, 300, 64, 129)
STD = 0.02


@pytest.mark.parametrize("shape", SHAPES, ids=lambda shape: "x".join(map(str, shape)))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_shape_whole_and_mixed(shape, dtype, model_root):
    heads, head_dim, intermediate, vocab, layers, page = shape
    hidden = heads * head_dim
    config = LlamaConfig(vocab_size=vocab, hidden_size=hidden, intermediate_size=intermediate,
                         num_hidden_layers=layers, num_attention_heads=heads,
                         num_key_value_heads=heads, head_dim=head_dim,
                         max_position_embeddings=320, rms_norm_eps=1e-5, rope_theta=10000.0)
    folder = os.path.join(model_root, "sweep_" + "_".join(map(str, shape)) + "_" + dtype)
    gain = (SCORE_SPREAD / (STD * STD * hidden)) ** 0.5
    write_random_model(folder, config, 3, std=STD, scale_std=0.1, storage_dtype=dtype,
                       gains={"q_proj": gain, "k_proj": gain})
    plain = plain_llama.PlainModel(folder, precision=dtype)
    requests = {f"r{index}": random_tokens(vocab, length, seed=50 + index)
                for index, length in enumerate(LENGTHS)}
    expected = {name: plain.logits(tokens) for name, tokens in requests.items()}
    if dtype == "float32":
        bounds = F32_TOL
    else:
        exact = plain_llama.PlainModel(folder, precision="float32")
        moved = max(float(np.abs(exact.logits(requests[name]) - expected[name]).max())
                    for name in ("r2", "r3"))
        bounds = dict(atol=0.8 * moved, rtol=BF16_TOL["rtol"])
    for what, steps in (("whole", traces.whole(requests)),
                        ("mixed", traces.mixed(requests, max_live=4, seed=3))):
        need = traces.live_token_need(steps, round_to=page)
        harness = Harness(folder, dtype, page, num_pages=need // page)
        positions = {}
        for step in steps:
            rows = traces.labels(step, positions)
            out = harness.run([(e["id"], e["tokens"], e["want"]) for e in step["entries"]])
            for name in step["end"]:
                harness.end(name)
            if rows:
                want = np.stack([expected[name][position] for name, position in rows])
                assert_close(out, want, f"{what} {shape} {dtype} step {step['step']}", **bounds)
        harness.cache.check()
        assert not harness.cache.live_requests()
