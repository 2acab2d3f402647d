"""A toy mixer with state of its own, defined here, registered, built and stepped without a
change to the framework's files.

The toy architecture alternates the framework's attention with a "decayed sum" mixer that
keeps one vector per request between steps (no pages), runs one block twice, and lets its
last attention layer read the cache of the first.  Its steps are compared with a plain
whole-sequence computation written here, under several ways of cutting.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import List, Mapping, Optional

import numpy as np
import pytest
import torch

import plain_llama as plain
from conftest import random_tokens
from engine_harness import Harness, assert_close
from helix_runtime_b200 import (ModelSpec, PartSpec, register_architecture, register_part,
                                write_random_model)
from helix_runtime_b200.cache import StateNeed
from helix_runtime_b200.config import BlockSpec, ScheduleEntry
from helix_runtime_b200.parts import Mixer
from helix_runtime_b200.weights import TensorRequest

pytestmark = pytest.mark.gpu

HIDDEN, HEADS, HEAD_DIM, INTER, VOCAB, POSITIONS = 48, 3, 16, 40, 97, 64
DECAY = 0.75


class DecayedSum(Mixer):
    """y_t = w * s_t with s_t = decay * s_{t-1} + x_t; s lives in the request's state slot."""

    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.decay = float(spec["decay"])
        self.name = spec.tensors["weight"]
        self.weight: Optional[torch.Tensor] = None

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.hidden_size,), torch.float32)

    def tensor_requests(self) -> List[TensorRequest]:
        return [TensorRequest(self.name, (self.hidden_size,), role="scale")]

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        self.weight = tensors[self.name].to(device=device, dtype=torch.float32)

    def forward(self, ctx, cache, x, residual) -> None:
        """Everything is computed from the step's DEVICE arrays with shapes that depend on
        the number of tokens and requests only, and nothing is read back to the host, so the
        same calls can be recorded into a CUDA graph and replayed while positions, slots and
        tokens change underneath.  s_j = decay^(i+1) * s_before + sum_{k<=i} decay^(i-k) x_k
        for the i-th token of a request in this step, as one masked matrix product."""
        n, requests = ctx.n_tokens, ctx.n_requests
        owner = ctx.token_request[:n].long()                       # request index per token
        start = ctx.request_start[:requests + 1].long()
        slot = ctx.request_slot[:requests].long()
        index = torch.arange(n, device=x.device)
        local = index - start[owner]                               # place within the request
        same = owner[:, None] == owner[None, :]
        earlier = index[None, :] <= index[:, None]
        power = (index[:, None] - index[None, :]).clamp(min=0).float()
        weights = torch.where(same & earlier, self.decay ** power, torch.zeros_like(power))
        before = cache.state.index_select(0, slot)                 # [requests, hidden]
        carried = (self.decay ** (local + 1).float())[:, None] * before.index_select(0, owner)
        states = weights @ x[:n].float() + carried
        residual[:n] += self.weight * states
        last = start[1:] - 1                                       # last token of each request
        cache.state.index_copy_(0, slot, states.index_select(0, last))


@dataclasses.dataclass(frozen=True)
class ToyConfig:
    decay: float = DECAY

    def to_dict(self):
        return {"architectures": ["ToyStateForCausalLM"], "model_type": "toy_state",
                "decay": self.decay}


def attention_spec(prefix: str) -> PartSpec:
    position = PartSpec("rotary", {"theta": 100.0, "head_dim": HEAD_DIM, "rotary_dim": HEAD_DIM,
                                   "pairing": "adjacent", "max_positions": POSITIONS})
    return PartSpec("paged_attention",
                    {"num_heads": HEADS, "num_kv_heads": HEADS, "head_dim": HEAD_DIM, "scale": None,
                     "window": None, "position": position, "checkpoint_pairing": "adjacent"},
                    {name: f"{prefix}.{name}" for name in ("q", "k", "v", "o")})


def block_spec(index: int, mixer: PartSpec) -> BlockSpec:
    return BlockSpec(
        arrangement="pre_norm",
        mixer_norm=PartSpec("rms", {"eps": 1e-5}, {"weight": f"b{index}.norm1"}),
        mixer=mixer,
        feed_forward_norm=PartSpec("rms", {"eps": 1e-5}, {"weight": f"b{index}.norm2"}),
        feed_forward=PartSpec("gated_mlp", {"intermediate_size": INTER, "activation": "silu"},
                              {name: f"b{index}.{name}" for name in ("gate", "up", "down")}))


def build_toy_spec(config: ToyConfig) -> ModelSpec:
    blocks = (block_spec(0, attention_spec("b0")),
              block_spec(1, PartSpec("decayed_sum", {"decay": config.decay}, {"weight": "b1.mix"})))
    # block 1 runs twice (two states), and the last entry re-reads the cache of entry 0
    schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1), ScheduleEntry(0, cache_from=0))
    return ModelSpec(
        architecture="ToyStateForCausalLM", hidden_size=HIDDEN, vocab_size=VOCAB,
        max_positions=POSITIONS,
        embedding=PartSpec("token_table", {"vocab_size": VOCAB}, {"weight": "embed"}),
        blocks=blocks, schedule=schedule,
        final_norm=PartSpec("rms", {"eps": 1e-5}, {"weight": "norm"}),
        lm_head=PartSpec("linear", {"vocab_size": VOCAB, "tied": False}, {"weight": "head"}))


register_part("mixer", "decayed_sum", DecayedSum)
register_architecture("ToyStateForCausalLM", lambda doc: ToyConfig(decay=float(doc["decay"])),
                      build_toy_spec, aliases=("toy_state",))


def plain_toy(tensors, tokens):
    """The toy model on one whole sequence, from the same formulas, in NumPy."""
    t = {name: value.float().numpy() for name, value in tensors.items()}
    hidden = t["embed"][np.asarray(tokens)]
    count = len(tokens)
    cosine, sine = plain.rope_table(count, HEAD_DIM, 100.0)

    def attention(x):
        q = plain.linear(x, t["b0.q"].T).reshape(count, HEADS, HEAD_DIM)
        k = plain.linear(x, t["b0.k"].T).reshape(count, HEADS, HEAD_DIM)
        v = plain.linear(x, t["b0.v"].T).reshape(count, HEADS, HEAD_DIM)
        q = plain.rope_adjacent(q, cosine, sine).transpose(1, 0, 2)
        k = plain.rope_adjacent(k, cosine, sine).transpose(1, 0, 2)
        return q, k, v.transpose(1, 0, 2)

    def mlp(index, x):
        return plain.linear(plain.swiglu(plain.linear(x, t[f"b{index}.gate"].T),
                                         plain.linear(x, t[f"b{index}.up"].T)), t[f"b{index}.down"].T)

    first_keys = None
    for entry, block in enumerate((0, 1, 1, 0)):
        normed = plain.rms_norm(hidden, t[f"b{block}.norm1"], 1e-5)
        if block == 0:
            q, k, v = attention(normed)
            if entry == 0:
                first_keys = (k, v)
            else:
                k, v = first_keys          # the last entry reads the first entry's cache
            context = plain.causal_attention(q, k, v).transpose(1, 0, 2).reshape(count, -1)
            hidden = hidden + plain.linear(context, t["b0.o"].T)
        else:
            state = np.zeros(HIDDEN, dtype=np.float32)
            out = np.zeros_like(hidden)
            for position in range(count):
                state = (state * np.float32(DECAY) + normed[position]).astype(np.float32)
                out[position] = t["b1.mix"] * state
            hidden = hidden + out
        normed = plain.rms_norm(hidden, t[f"b{block}.norm2"], 1e-5)
        hidden = (hidden + mlp(block, normed)).astype(np.float32)
    return plain.linear(plain.rms_norm(hidden, t["norm"], 1e-5), t["head"].T)


def test_toy_architecture_with_state_steps_like_its_plain_form(tmp_path):
    folder = str(tmp_path / "toy")
    write_random_model(folder, ToyConfig(), seed=3, std=0.08, scale_std=0.2,
                       storage_dtype="float32")
    with open(os.path.join(folder, "config.json")) as source:
        assert json.load(source)["architectures"] == ["ToyStateForCausalLM"]
    from helix_runtime_b200.weights import Checkpoint
    checkpoint = Checkpoint(folder)
    tensors = {name: checkpoint.read(name) for name in checkpoint.names()}
    harness = Harness(folder, "float32", page_size=4, num_pages=40, max_requests=3, max_tokens=128)
    kv_needs, state_needs = harness.model.cache_needs()
    assert sorted(kv_needs) == [0] and sorted(state_needs) == [1, 2]    # entry 3 owns nothing
    assert len(harness.cache.groups) == 1 and len(harness.cache.groups[0].entries) == 1

    a = random_tokens(VOCAB, 40, seed=1)
    b = random_tokens(VOCAB, 23, seed=2)
    expected_a, expected_b = plain_toy(tensors, a), plain_toy(tensors, b)
    tol = dict(atol=5e-5, rtol=1e-4)
    assert_close(harness.whole("a", a), expected_a, "whole a", **tol)
    # the same two requests cut into portions and single tokens, side by side; b starts in the
    # state slot that a's first run left behind, which must have been cleared
    out = harness.run([("b", b[:5], range(5)), ("a", a[:17], range(17))])
    assert_close(out, np.concatenate([expected_b[:5], expected_a[:17]]), "first portions", **tol)
    out = harness.run([("a", a[17:19], range(2))])
    assert_close(out, expected_a[17:19], "a alone", **tol)
    for position in range(5, 23):
        step = [("b", [b[position]], [0])]
        if 19 + (position - 5) < 40:
            step.append(("a", [a[19 + position - 5]], [0]))
        out = harness.run(step)
        assert_close(out[:1], expected_b[position:position + 1], f"b decode {position}", **tol)
        if len(step) == 2:
            assert_close(out[1:], expected_a[19 + position - 5:20 + position - 5],
                         f"a decode beside b {position}", **tol)
    harness.end("a")
    harness.end("b")
    harness.cache.check()


@pytest.mark.parametrize("cuda_graphs", [False, True])
def test_state_of_a_mixer_survives_graph_replay(tmp_path, cuda_graphs):
    """The toy model through the engine itself: admission, prompt portions, then decode steps
    that are recorded into CUDA graphs and queued ahead of one another.  The mixer's state is
    read and written through the device arrays of the step, so the recorded launches serve
    every later step; the tokens equal the plain form's."""
    from helix_runtime_b200 import Engine
    from helix_runtime_b200.weights import Checkpoint
    folder = str(tmp_path / "toy")
    write_random_model(folder, ToyConfig(), seed=3, std=0.08, scale_std=0.2,
                       storage_dtype="float32")
    checkpoint = Checkpoint(folder)
    tensors = {name: checkpoint.read(name) for name in checkpoint.names()}
    engine = Engine.from_pretrained(folder, dtype="float32", page_size=4, max_running_requests=3,
                                    max_tokens_per_iteration=16, max_prefill_chunk=7,
                                    cuda_graphs=cuda_graphs)
    prompts = [random_tokens(VOCAB, n, seed=20 + n) for n in (13, 3, 22, 6)]
    results = engine.generate(prompts, max_new_tokens=30)
    if cuda_graphs:
        assert engine.graphs.captures > 0 and engine.graphs.replays > 20
        assert engine.steps_queued_ahead > 0
    for prompt, result in zip(prompts, results):
        assert len(result.generated_tokens) == 30
        logits = plain_toy(tensors, prompt + result.generated_tokens[:-1])
        for index, token in enumerate(result.generated_tokens):
            row = logits[len(prompt) + index - 1]
            assert row[token] >= row.max() - 1e-4, f"token {index}"
    engine.cache.check()


@pytest.mark.parametrize("cuda_graphs", [False, True])
def test_the_next_turn_of_a_conversation_starts_from_the_kept_state(tmp_path, cuda_graphs):
    """Prefix sharing for a model with per-request state.  The scheduler ends a prompt portion
    at the prompt's last page boundary, the engine copies the mixers' state as that step
    leaves it, and the prefix index keeps the copy with the pages; the next turn (the first
    prompt, its answer and more) adopts pages AND state and computes only what is new.  Its
    tokens equal the plain form's, which knows nothing of any of this."""
    from helix_runtime_b200 import Engine
    from helix_runtime_b200.weights import Checkpoint
    folder = str(tmp_path / "toy")
    write_random_model(folder, ToyConfig(), seed=3, std=0.08, scale_std=0.2,
                       storage_dtype="float32")
    checkpoint = Checkpoint(folder)
    tensors = {name: checkpoint.read(name) for name in checkpoint.names()}
    engine = Engine.from_pretrained(folder, dtype="float32", page_size=4, max_running_requests=3,
                                    max_tokens_per_iteration=16, max_prefill_chunk=7,
                                    cuda_graphs=cuda_graphs, prefix_cache_entries=4,
                                    poison_free_pages=True)

    def check(prompt, result):
        logits = plain_toy(tensors, prompt + result.generated_tokens[:-1])
        for index, token in enumerate(result.generated_tokens):
            row = logits[len(prompt) + index - 1]
            assert row[token] >= row.max() - 1e-4, f"token {index}"

    first = random_tokens(VOCAB, 14, seed=31)            # its prefix: 12 tokens
    one = engine.generate([first], max_new_tokens=6)[0]
    check(first, one)
    second = first + one.generated_tokens + random_tokens(VOCAB, 5, seed=32)      # 25 tokens
    other = random_tokens(VOCAB, 9, seed=33)             # runs beside it, shares nothing
    two, beside = engine.generate([second, other], max_new_tokens=8)
    check(second, two)
    check(other, beside)
    assert engine.request(two.request_id).reused_tokens == 12
    assert engine.request(beside.request_id).reused_tokens == 0
    stats = engine.stats()["prefix"]
    assert stats["hits"] == 1 and stats["not_kept"] == 0 and stats["published"] == 3
    # the third turn goes on from the second: 24 of its tokens are there already
    third = second + two.generated_tokens + random_tokens(VOCAB, 3, seed=34)
    three = engine.generate([third], max_new_tokens=5)[0]
    check(third, three)
    assert engine.request(three.request_id).reused_tokens == 24
    engine.cache.check()
    engine.prefix.clear()
    engine.cache.check()
    assert all(group.pool.pages_in_use == 0 for group in engine.cache.groups)
