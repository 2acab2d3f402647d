"""The engine's model, cache and step function against the plain implementation, in process.

Every way of cutting the same requests into steps must give the plain implementation's
logits at every position: whole, tail decoded one by one, portions of changing size, and
mixed batches over a pool so small that pages are used again (free pages are filled with
NaN, so reading a page that was given back shows at once).
"""
from __future__ import annotations

import os

import numpy as np
import pytest

import traces
from conftest import random_tokens
from engine_harness import Harness, assert_close, tolerance
from tiny_configs import PAGE_SIZE, tiny_config

pytestmark = pytest.mark.gpu

LENGTHS = {"A": (5, 17, 31, 77), "B": (1, 9, 40, 64, 100), "C": (3, 20, 70, 150, 300)}
# C: the shapes of the fast kernels (see tiny_configs), in bfloat16 where they run
CASES = [("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("B", "bfloat16"),
         ("C", "bfloat16")]


def make_requests(name: str, extra: int = 0):
    vocab = tiny_config(name).vocab_size
    return {f"r{index}": random_tokens(vocab, length + extra, seed=1000 * (ord(name)) + index)
            for index, length in enumerate(LENGTHS[name])}


def replay(harness: Harness, steps, expected, dtype: str, what: str, model_name: str = ""):
    positions = {}
    for step in steps:
        rows = traces.labels(step, positions)
        out = harness.run([(e["id"], e["tokens"], e["want"]) for e in step["entries"]])
        for name in step["end"]:
            harness.end(name)
        if rows:
            want = np.stack([expected[name][position] for name, position in rows])
            assert_close(out, want, f"{what} step {step['step']} rows {rows[:4]}...",
                         **tolerance(dtype, model_name))
    harness.cache.check()
    assert not harness.cache.live_requests()


@pytest.fixture(scope="module")
def expectations(plain_models):
    cache = {}

    def get(name: str, dtype: str, extra: int = 0):
        key = (name, dtype, extra)
        if key not in cache:
            plain = plain_models(name, dtype)
            cache[key] = {request: plain.logits(tokens)
                          for request, tokens in make_requests(name, extra).items()}
        return cache[key]
    return get


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_requests(name, dtype, folders, expectations):
    harness = Harness(folders(name, dtype), dtype, PAGE_SIZE[name], num_pages=64)
    replay(harness, traces.whole(make_requests(name)), expectations(name, dtype), dtype,
           f"whole {name} {dtype}", name)


@pytest.mark.parametrize("name,dtype", CASES)
def test_tail_decoded_one_by_one(name, dtype, folders, expectations):
    harness = Harness(folders(name, dtype), dtype, PAGE_SIZE[name], num_pages=64)
    replay(harness, traces.tail_decoded(make_requests(name, extra=20)),
           expectations(name, dtype, 20), dtype, f"tail {name} {dtype}", name)


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions_of_changing_size(name, dtype, folders, expectations):
    harness = Harness(folders(name, dtype), dtype, PAGE_SIZE[name], num_pages=64)
    replay(harness, traces.chunked(make_requests(name, extra=20)),
           expectations(name, dtype, 20), dtype, f"portions {name} {dtype}", name)


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_batches_with_page_reuse(name, dtype, folders, expectations):
    requests = make_requests(name, extra=20)
    # twice the same requests under new names, so that later ones run in recycled pages
    doubled = dict(requests)
    doubled.update({f"again_{key}": value for key, value in requests.items()})
    expected = dict(expectations(name, dtype, 20))
    expected.update({f"again_{key}": value for key, value in expectations(name, dtype, 20).items()})
    steps = traces.mixed(doubled, max_live=4, seed=7)
    page = PAGE_SIZE[name]
    need = traces.live_token_need(steps, round_to=page)
    harness = Harness(folders(name, dtype), dtype, page, num_pages=need // page)
    replay(harness, steps, expected, dtype, f"mixed {name} {dtype}", name)
    group = harness.cache.groups[0]
    assert group.pool.reuse_count > 0, "the pool was large enough that no page was used again"


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A", "bfloat16")])
def test_long_decoding_to_the_last_position(name, dtype, folders, plain_models):
    config = tiny_config(name)
    tokens = random_tokens(config.vocab_size, config.max_position_embeddings, seed=5)
    expected = plain_models(name, dtype).logits(tokens)
    harness = Harness(folders(name, dtype), dtype, PAGE_SIZE[name], num_pages=32, split_keys=32)
    out = harness.run([("long", tokens[:3], [0, 1, 2])])
    assert_close(out, expected[:3], "prompt", **tolerance(dtype))
    for position in range(3, len(tokens)):
        out = harness.run([("long", [tokens[position]], [0])])
        assert_close(out, expected[position:position + 1], f"decode position {position}",
                     **tolerance(dtype))
    harness.end("long")
    harness.cache.check()


@pytest.mark.parametrize("name,dtype", CASES)
def test_first_tokens_of_a_sequence(name, dtype, folders, plain_models):
    vocab = tiny_config(name).vocab_size
    plain = plain_models(name, dtype)
    harness = Harness(folders(name, dtype), dtype, PAGE_SIZE[name], num_pages=16)
    for length in (1, 2, 3):
        tokens = random_tokens(vocab, length, seed=length)
        assert_close(harness.whole(f"w{length}", tokens), plain.logits(tokens),
                     f"whole prompt of {length}", **tolerance(dtype, name))
    tokens = random_tokens(vocab, 4, seed=9)
    expected = plain.logits(tokens)
    for position, token in enumerate(tokens):
        out = harness.run([("one", [token], [0])])
        assert_close(out, expected[position:position + 1], f"token {position} alone",
                     **tolerance(dtype, name))
    harness.end("one")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_key_among_hundreds(dtype, folders, plain_models):
    """Sharp attention (query/key projections scaled up) over 250 positions of tiny B: the
    decoded tail must still see every far key, across many pages and several key splits."""
    config = tiny_config("B")
    tokens = random_tokens(config.vocab_size, 250, seed=77)
    expected = plain_models("B", dtype).logits(tokens)
    harness = Harness(folders("B", dtype), dtype, PAGE_SIZE["B"], num_pages=20, split_keys=64)
    out = harness.run([("far", tokens[:200], range(200))])
    assert_close(out, expected[:200], "prompt of 200", **tolerance(dtype))
    for position in range(200, 250):
        out = harness.run([("far", [tokens[position]], [0])])
        assert_close(out, expected[position:position + 1], f"decode position {position}",
                     **tolerance(dtype))
    harness.end("far")


def test_wanting_nothing_returns_nothing_and_still_fills_the_cache(folders, plain_models):
    tokens = random_tokens(tiny_config("A").vocab_size, 20, seed=3)
    expected = plain_models("A", "float32").logits(tokens)
    harness = Harness(folders("A", "float32"), "float32", PAGE_SIZE["A"], num_pages=16)
    assert harness.run([("q", tokens[:19], [])]) is None
    out = harness.run([("q", tokens[19:], [0])])
    assert_close(out, expected[19:], "after a silent prompt", **tolerance("float32"))
    harness.end("q")


def test_llama_7b_layer_sizes_bfloat16_against_the_float32_path():
    """Two layers with the layer sizes of the benchmark model (hidden 4096, 32 heads of 128,
    intermediate 11008, vocabulary 32000): the bfloat16 engine (tcgen05 products on tiled
    weights, tcgen05 prompt attention, streaming decode attention, split-K weight streams)
    against the engine's own float32 path on the same (rounded) weights: CUDA-core kernels, no
    kernel in common.  A prompt in two portions, then token by token.  The plain
    implementation is too slow at this size; the float32 path is what the other tests hold
    against it.

    This is a detector of gross errors, not of rounding: a wrong tile, page, head or split
    changes the logits of the rows it touches by about their spread (1.3 here).  What
    bfloat16 storage of the activations does to them is far smaller but not tiny: about a
    hundredth of the spread (0.017 root mean square, 0.08 at most among 800,000 values), the
    same for every row, prompt or decoded.  The bounds are twice that."""
    import torch

    from helix_runtime_b200 import LlamaConfig, random_model
    from helix_runtime_b200.cache.manager import CacheManager
    from helix_runtime_b200.engine.step import StepEntry, StepFunction

    config = LlamaConfig(vocab_size=32000, hidden_size=4096, intermediate_size=11008,
                         num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=32,
                         head_dim=128, max_position_embeddings=1024, rms_norm_eps=1e-5,
                         rope_theta=10000.0)
    tokens = random_tokens(32000, 400, seed=77)
    results = {}
    for dtype in ("float32", "bfloat16"):
        model = random_model(config, 0, dtype, torch.device("cuda:0"))
        if dtype == "float32":
            # the same weights as the bfloat16 model holds: rounded, then kept in 32 bits
            matrices = [model.embedding.table, model.lm_head.weight.matrix]
            for block in model.blocks:
                matrices += [block.mixer.w_qkv.matrix, block.mixer.w_o.matrix,
                             block.feed_forward.w_gate_up.matrix, block.feed_forward.w_down.matrix]
            for matrix in matrices:
                matrix.copy_(matrix.to(torch.bfloat16).to(torch.float32))
        kv, state = model.cache_needs()
        cache = CacheManager(kv, state, 16, 64, 2, 1024, model.dtype, torch.device("cuda:0"),
                             poison=True)
        step = StepFunction(model, cache, max_tokens=512, max_requests=2)
        cache.admit("r")
        rows = []
        rows.append(step.run([StepEntry("r", tokens[:300], [0, 150, 299])]).float().cpu().numpy().copy())
        rows.append(step.run([StepEntry("r", tokens[300:380], [0, 79])]).float().cpu().numpy().copy())
        for position in range(380, 400):
            rows.append(step.run([StepEntry("r", [tokens[position]], [0])]).float().cpu().numpy().copy())
        results[dtype] = np.concatenate(rows)
        cache.release("r")
        cache.check()
        del model, cache, step
        torch.cuda.empty_cache()
    exact, fast = results["float32"], results["bfloat16"]
    assert np.isfinite(fast).all()
    spread = float(exact.std())
    assert 0.3 < spread < 3.0, spread
    difference = np.abs(exact - fast)
    per_row = np.sqrt((difference ** 2).mean(axis=-1))
    assert (per_row < 0.025 * spread).all(), \
        f"root mean square difference per row {np.round(per_row, 4).tolist()} (spread {spread})"
    assert difference.max() < 0.12 * spread, f"largest difference {difference.max()}"
    # and the two agree on which token is best where the best is clear
    top2 = np.sort(exact, axis=-1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 0.1
    assert (np.argmax(exact, axis=-1)[clear] == np.argmax(fast, axis=-1)[clear]).all()


@pytest.fixture(scope="module")
def llama_7b_layer(model_root):
    """One layer of the benchmark model's sizes as a folder, a sequence, and what the plain
    implementation makes of it in float32 and with activations rounded to bfloat16."""
    import plain_llama
    from helix_runtime_b200 import LlamaConfig, write_random_model
    from tiny_configs import SCORE_SPREAD

    config = LlamaConfig(vocab_size=32000, hidden_size=4096, intermediate_size=11008,
                         num_hidden_layers=1, num_attention_heads=32, num_key_value_heads=32,
                         head_dim=128, max_position_embeddings=512, rms_norm_eps=1e-5,
                         rope_theta=10000.0)
    folder = os.path.join(model_root, "llama_7b_layer")
    gain = (SCORE_SPREAD / (0.02 * 0.02 * 4096)) ** 0.5
    write_random_model(folder, config, 5, std=0.02, scale_std=0.1, storage_dtype="bfloat16",
                       gains={"q_proj": gain, "k_proj": gain})
    tokens = random_tokens(32000, 320, seed=78)
    plain = plain_llama.PlainModel(folder, precision="float32")
    exact = plain.logits(tokens)
    plain.precision = "bfloat16"
    return folder, tokens, {"float32": exact, "bfloat16": plain.logits(tokens)}


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_llama_7b_layer_sizes_against_the_plain_implementation(dtype, llama_7b_layer):
    """One layer with the layer sizes of the benchmark model (hidden 4096, 32 heads of 128,
    intermediate 11008, vocabulary 32000) against the plain implementation, which shares
    nothing with the engine: split-K over depths of 4096 and 11008, the 32,000-row output head,
    128-wide heads, tiled weights.  A prompt in two portions, then twenty tokens one by one.
    The bfloat16 bound is measured, as for the other shapes: 0.8 of what rounding the
    activations to bfloat16 does to this model's logits in the plain implementation."""
    from engine_harness import BF16_TOL, F32_TOL, Harness

    folder, tokens, logits = llama_7b_layer
    expected = logits[dtype]
    if dtype == "float32":
        # the tiny models' bound (2e-5 + 1e-4 |x|) is 1e-4 of their logits' spread of 0.2 plus
        # 1e-4 of the value; the same rule for this model, whose logits spread over 1.3 and
        # whose float32 sums have 4,096 to 11,008 terms
        spread = float(expected.std())
        assert 0.5 < spread < 3.0, spread
        bounds = dict(atol=F32_TOL["atol"] * spread / 0.2, rtol=F32_TOL["rtol"])
    else:
        moved = float(np.abs(logits["float32"] - expected).max())
        assert 1e-3 < moved < 0.5, moved
        bounds = dict(atol=0.8 * moved, rtol=BF16_TOL["rtol"])
    harness = Harness(folder, dtype, 16, num_pages=24, max_requests=1, max_tokens=256)
    out = harness.run([("r", tokens[:180], [0, 100, 179])])
    assert_close(out, expected[[0, 100, 179]], f"first portion {dtype}", **bounds)
    out = harness.run([("r", tokens[180:300], [0, 119])])
    assert_close(out, expected[[180, 299]], f"second portion {dtype}", **bounds)
    for position in range(300, 320):
        out = harness.run([("r", [tokens[position]], [0])])
        assert_close(out, expected[[position]], f"decoded token at {position} {dtype}", **bounds)
    harness.end("r")
    harness.cache.check()
