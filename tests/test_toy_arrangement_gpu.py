"""Block arrangements registered from outside the framework, and a pool sized for a window.

The toy architecture here has two arrangements of its own, registered by this file: a
parallel residual (one norm feeds the mixer and the feed-forward, both add into the stream)
and a block that has a mixer and no feed-forward at all.  Every layer's attention is
windowed, so a request never holds more pages than its window needs: the engine must accept
and run a prompt that is longer than the whole pool.  Logits and generated tokens are compared
with a plain whole-sequence computation written here.  Nobody's model; it shows what the
interfaces carry.
"""
from __future__ import annotations

import dataclasses

import numpy as np
import pytest

import plain_llama as plain
from conftest import random_tokens
from engine_harness import Harness, assert_close
from helix_runtime_b200 import (Engine, ModelSpec, PartSpec, register_architecture,
                                register_arrangement, write_random_model)
from helix_runtime_b200.config import BlockSpec, ScheduleEntry
from helix_runtime_b200.weights import Checkpoint

pytestmark = pytest.mark.gpu

HIDDEN, HEADS, HEAD_DIM, INTER, VOCAB, POSITIONS = 32, 2, 16, 24, 61, 96
WINDOW, PAGE = 12, 4


def parallel_residual(block, ctx, cache, residual, normed) -> None:
    """x += mixer(norm(x)) + ff(norm(x)): both read the same normed rows."""
    block.mixer_norm.forward(ctx, residual, normed)
    block.mixer.forward(ctx, cache, normed, residual)
    block.feed_forward.forward(ctx, normed, residual)


def mixer_only(block, ctx, cache, residual, normed) -> None:
    block.mixer_norm.forward(ctx, residual, normed)
    block.mixer.forward(ctx, cache, normed, residual)


register_arrangement("toy_parallel_residual", parallel_residual)
register_arrangement("toy_mixer_only", mixer_only)


@dataclasses.dataclass(frozen=True)
class ToyParallelConfig:
    window: int = WINDOW

    def to_dict(self):
        return {"architectures": ["ToyParallelForCausalLM"], "model_type": "toy_parallel",
                "window": self.window}


def attention(prefix: str, window: int) -> PartSpec:
    rotary = PartSpec("rotary", {"theta": 80.0, "head_dim": HEAD_DIM, "rotary_dim": HEAD_DIM,
                                 "pairing": "adjacent", "max_positions": POSITIONS})
    return PartSpec("paged_attention",
                    {"num_heads": HEADS, "num_kv_heads": HEADS, "head_dim": HEAD_DIM, "scale": None,
                     "window": window, "position": rotary, "checkpoint_pairing": "adjacent"},
                    {name: f"{prefix}.{name}" for name in ("q", "k", "v", "o")})


def build_spec(config: ToyParallelConfig) -> ModelSpec:
    blocks = (
        BlockSpec("toy_parallel_residual",
                  mixer_norm=PartSpec("rms", {"eps": 1e-5}, {"weight": "b0.norm"}),
                  mixer=attention("b0", config.window),
                  feed_forward=PartSpec("gated_mlp", {"intermediate_size": INTER,
                                                      "activation": "silu"},
                                        {name: f"b0.{name}" for name in ("gate", "up", "down")})),
        BlockSpec("toy_mixer_only",
                  mixer_norm=PartSpec("rms", {"eps": 1e-5}, {"weight": "b1.norm"}),
                  mixer=attention("b1", config.window)))
    return ModelSpec(
        architecture="ToyParallelForCausalLM", hidden_size=HIDDEN, vocab_size=VOCAB,
        max_positions=POSITIONS,
        embedding=PartSpec("token_table", {"vocab_size": VOCAB}, {"weight": "embed"}),
        blocks=blocks, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)),
        final_norm=PartSpec("rms", {"eps": 1e-5}, {"weight": "norm"}),
        lm_head=PartSpec("linear", {"vocab_size": VOCAB, "tied": False}, {"weight": "head"}))


register_architecture("ToyParallelForCausalLM",
                      lambda doc: ToyParallelConfig(window=int(doc["window"])), build_spec,
                      aliases=("toy_parallel",))


def plain_toy(tensors, tokens):
    t = {name: value.float().numpy() for name, value in tensors.items()}
    hidden = t["embed"][np.asarray(tokens)]
    count = len(tokens)
    cosine, sine = plain.rope_table(count, HEAD_DIM, 80.0)

    def attend(prefix, x):
        q, k, v = (plain.linear(x, t[f"{prefix}.{name}"].T).reshape(count, HEADS, HEAD_DIM)
                   for name in ("q", "k", "v"))
        q = plain.rope_adjacent(q, cosine, sine).transpose(1, 0, 2)
        k = plain.rope_adjacent(k, cosine, sine).transpose(1, 0, 2)
        context = plain.causal_attention(q, k, v.transpose(1, 0, 2), window=WINDOW)
        return plain.linear(context.transpose(1, 0, 2).reshape(count, -1), t[f"{prefix}.o"].T)

    for block in (0, 1, 0):
        normed = plain.rms_norm(hidden, t[f"b{block}.norm"], 1e-5)
        update = attend(f"b{block}", normed)
        if block == 0:
            update = update + plain.linear(
                plain.swiglu(plain.linear(normed, t["b0.gate"].T), plain.linear(normed, t["b0.up"].T)),
                t["b0.down"].T)
        hidden = (hidden + update).astype(np.float32)
    return plain.linear(plain.rms_norm(hidden, t["norm"], 1e-5), t["head"].T)


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    folder = str(tmp_path_factory.mktemp("toy_parallel") / "model")
    write_random_model(folder, ToyParallelConfig(), seed=4, std=0.1, scale_std=0.2,
                       storage_dtype="float32")
    checkpoint = Checkpoint(folder)
    return folder, {name: checkpoint.read(name) for name in checkpoint.names()}


def test_arrangements_registered_here_step_like_their_plain_form(toy):
    folder, tensors = toy
    harness = Harness(folder, "float32", page_size=PAGE, num_pages=30, max_requests=2,
                      max_tokens=128)
    assert [block.arrangement for block in harness.model.blocks] == \
        ["toy_parallel_residual", "toy_mixer_only"]
    assert harness.model.blocks[1].feed_forward is None
    a = random_tokens(VOCAB, 50, seed=1)
    b = random_tokens(VOCAB, 21, seed=2)
    expected_a, expected_b = plain_toy(tensors, a), plain_toy(tensors, b)
    tol = dict(atol=5e-5, rtol=1e-4)
    assert_close(harness.whole("a", a), expected_a, "whole", **tol)
    out = harness.run([("a", a[:19], range(19)), ("b", b[:2], range(2))])
    assert_close(out, np.concatenate([expected_a[:19], expected_b[:2]]), "portions", **tol)
    out = harness.run([("b", b[2:], range(19)), ("a", a[19:20], [0])])
    assert_close(out, np.concatenate([expected_b[2:], expected_a[19:20]]), "mixed", **tol)
    for position in range(20, 50):
        out = harness.run([("a", [a[position]], [0])])
        assert_close(out, expected_a[position:position + 1], f"decode {position}", **tol)
    harness.end("a")
    harness.end("b")
    harness.cache.check()
    with pytest.raises(ValueError, match="unknown block arrangement 'post_norm'; known: .*pre_norm"):
        from helix_runtime_b200.models import Block
        Block(BlockSpec("post_norm", mixer_norm=PartSpec("rms", {"eps": 1e-5}, {"weight": "n"}),
                        mixer=attention("b0", WINDOW)), HIDDEN)


@pytest.mark.parametrize("cuda_graphs", [False, True])
def test_a_pool_sized_for_the_window_runs_a_prompt_longer_than_the_pool(toy, cuda_graphs):
    """Five pages of four keys hold a window of twelve and the page being filled, nothing
    more: the prompt of forty tokens is fed in portions as pages come back, and decoding goes
    on to eighty positions, four times the pool."""
    folder, tensors = toy
    pool = WINDOW // PAGE + 2
    engine = Engine.from_pretrained(folder, dtype="float32", page_size=PAGE, num_pages=pool,
                                    max_running_requests=1, max_tokens_per_iteration=64,
                                    cuda_graphs=cuda_graphs, poison_free_pages=True)
    prompt = random_tokens(VOCAB, 40, seed=3)
    assert len(prompt) > pool * PAGE
    result = engine.generate([prompt], max_new_tokens=40)[0]
    assert len(result.generated_tokens) == 40 and result.cached_token_count == 79
    tokens = list(prompt)
    logits = plain_toy(tensors, prompt + result.generated_tokens[:-1])
    for index, token in enumerate(result.generated_tokens):
        row = logits[len(prompt) + index - 1]
        assert row[token] >= row.max() - 1e-4, f"token {index}"
    stats = engine.stats()["cache"]["groups"][0]
    assert stats["pages"] == pool and stats["reuses"] > 10 and stats["peak_pages_in_use"] <= pool
    assert engine.stats()["scheduler"]["preemptions"] == 0
    engine.cache.check()
    # what needs more than the window's pages at once is still refused: a group that keeps
    # every key would need 20 pages for this request
    assert engine.cache.pages_needed_alone(79) == [4]
