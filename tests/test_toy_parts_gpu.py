"""Other toy parts, defined here and registered from outside the framework: a feed-forward
with routing (top-1 of several small gated experts), a position encoding that is not rotary
(a learned vector per position added to queries and keys), and an architecture that mixes
them with the framework's own parts: full attention beside windowed attention (two cache
groups), a block that runs twice.  Its steps are compared with a plain whole-sequence
computation written here, under several ways of cutting.  None of these parts is anybody's
model; they show what the interfaces carry.
"""
from __future__ import annotations

import dataclasses
from typing import List, Mapping, Optional

import numpy as np
import pytest
import torch

import plain_llama as plain
from conftest import random_tokens
from engine_harness import Harness, assert_close
from helix_runtime_b200 import (ModelSpec, PartSpec, register_architecture, register_part,
                                write_random_model)
from helix_runtime_b200.config import BlockSpec, ScheduleEntry
from helix_runtime_b200.ops import library as ops
from helix_runtime_b200.parts import FeedForward, PositionEncoding
from helix_runtime_b200.weights import Checkpoint, TensorRequest

pytestmark = pytest.mark.gpu

HIDDEN, HEADS, HEAD_DIM, INTER, VOCAB, POSITIONS = 40, 5, 8, 24, 89, 48
EXPERTS, WINDOW = 3, 6


class LearnedQueryKeyBias(PositionEncoding):
    """q_t += b[pos_t], k_t += b[pos_t] for every head; values untouched; then the append."""

    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.head_dim = int(spec["head_dim"])
        self.max_positions = int(spec["max_positions"])
        self.name = spec.tensors["table"]
        self.table: Optional[torch.Tensor] = None
        self.nothing: Optional[torch.Tensor] = None

    def tensor_requests(self) -> List[TensorRequest]:
        return [TensorRequest(self.name, (self.max_positions, self.head_dim), role="scale")]

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        self.table = tensors[self.name].to(device=device, dtype=torch.float32)
        self.nothing = torch.zeros((1, 1), dtype=torch.float32, device=device)

    def apply(self, ctx, cache, qkv, heads, kv_heads, accum=None) -> None:
        n = ctx.n_tokens
        if accum is not None:      # the projection arrives in a float32 accumulator: take it over
            qkv[:n] = accum[:n].to(qkv.dtype)
            accum[:n].zero_()
        rows = qkv[:n].view(n, heads + 2 * kv_heads, self.head_dim)
        bias = self.table[ctx.positions[:n].long()]
        rows[:, :heads + kv_heads] = (rows[:, :heads + kv_heads].float() +
                                      bias[:, None, :]).to(qkv.dtype)
        write = cache.owns and cache.keys is not None
        # the framework's append kernel with nothing to rotate
        ops.rope_append(qkv, ctx.positions, ctx.token_request, ctx.request_slot,
                        cache.block_tables, cache.keys if write else None,
                        cache.values if write else None, self.nothing, self.nothing, n, heads,
                        kv_heads, self.head_dim, 0, 0, cache.page_size, cache.num_pages, ctx.status)


class RoutedMlp(FeedForward):
    """Router logits in float32, softmax, the best expert only, weighted by its probability.
    It asks the device which rows chose an expert (``nonzero``), so it cannot be recorded
    into a CUDA graph and says so; the engine then runs this model's steps eagerly."""

    graph_safe = False

    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.experts = int(spec["experts"])
        self.intermediate = int(spec["intermediate_size"])
        self.prefix = spec.tensors["prefix"]
        self.router = None
        self.gate, self.up, self.down = [], [], []

    def tensor_requests(self) -> List[TensorRequest]:
        h, i = self.hidden_size, self.intermediate
        requests = [TensorRequest(f"{self.prefix}.router", (self.experts, h), role="scale")]
        for e in range(self.experts):
            requests += [TensorRequest(f"{self.prefix}.{e}.gate", (i, h)),
                         TensorRequest(f"{self.prefix}.{e}.up", (i, h)),
                         TensorRequest(f"{self.prefix}.{e}.down", (h, i))]
        return requests

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        self.router = tensors[f"{self.prefix}.router"].to(device=device, dtype=torch.float32)
        for name, target in (("gate", self.gate), ("up", self.up), ("down", self.down)):
            target[:] = [tensors[f"{self.prefix}.{e}.{name}"].to(device=device, dtype=torch.float32)
                         for e in range(self.experts)]

    def forward(self, ctx, x, residual) -> None:
        n = ctx.n_tokens
        tokens = x[:n].float()
        probabilities = torch.softmax(tokens @ self.router.T, dim=-1)
        weight, choice = probabilities.max(dim=-1)
        for e in range(self.experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            picked = tokens[rows]
            hidden = torch.nn.functional.silu(picked @ self.gate[e].T) * (picked @ self.up[e].T)
            residual.index_add_(0, rows, (hidden @ self.down[e].T) * weight[rows, None])


@dataclasses.dataclass(frozen=True)
class ToyRoutedConfig:
    window: int = WINDOW

    def to_dict(self):
        return {"architectures": ["ToyRoutedForCausalLM"], "model_type": "toy_routed",
                "window": self.window}


def attention_spec(prefix: str, position: PartSpec, window) -> PartSpec:
    return PartSpec("paged_attention",
                    {"num_heads": HEADS, "num_kv_heads": HEADS, "head_dim": HEAD_DIM, "scale": None,
                     "window": window, "position": position, "checkpoint_pairing": "adjacent"},
                    {name: f"{prefix}.{name}" for name in ("q", "k", "v", "o")})


def build_spec(config: ToyRoutedConfig) -> ModelSpec:
    learned = PartSpec("learned_qk_bias", {"head_dim": HEAD_DIM, "max_positions": POSITIONS},
                       {"table": "b0.positions"})
    rotary = PartSpec("rotary", {"theta": 50.0, "head_dim": HEAD_DIM, "rotary_dim": HEAD_DIM,
                                 "pairing": "adjacent", "max_positions": POSITIONS})

    def norms(index):
        return (PartSpec("rms", {"eps": 1e-5}, {"weight": f"b{index}.norm1"}),
                PartSpec("rms", {"eps": 1e-5}, {"weight": f"b{index}.norm2"}))

    blocks = (
        BlockSpec("pre_norm", norms(0)[0], attention_spec("b0", learned, None), norms(0)[1],
                  PartSpec("routed_mlp", {"experts": EXPERTS, "intermediate_size": INTER},
                           {"prefix": "b0.experts"})),
        BlockSpec("pre_norm", norms(1)[0], attention_spec("b1", rotary, config.window), norms(1)[1],
                  PartSpec("gated_mlp", {"intermediate_size": INTER, "activation": "silu"},
                           {name: f"b1.{name}" for name in ("gate", "up", "down")})))
    return ModelSpec(
        architecture="ToyRoutedForCausalLM", hidden_size=HIDDEN, vocab_size=VOCAB,
        max_positions=POSITIONS,
        embedding=PartSpec("token_table", {"vocab_size": VOCAB}, {"weight": "embed"}),
        blocks=blocks, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)),
        final_norm=PartSpec("rms", {"eps": 1e-5}, {"weight": "norm"}),
        lm_head=PartSpec("linear", {"vocab_size": VOCAB, "tied": False}, {"weight": "head"}))


register_part("position", "learned_qk_bias", LearnedQueryKeyBias)
register_part("feed_forward", "routed_mlp", RoutedMlp)
register_architecture("ToyRoutedForCausalLM", lambda doc: ToyRoutedConfig(window=int(doc["window"])),
                      build_spec, aliases=("toy_routed",))


def plain_toy(tensors, tokens):
    """The toy model on one whole sequence, from the same formulas, in NumPy."""
    t = {name: value.float().numpy() for name, value in tensors.items()}
    hidden = t["embed"][np.asarray(tokens)]
    count = len(tokens)
    cosine, sine = plain.rope_table(count, HEAD_DIM, 50.0)

    def heads_of(x, name):
        return plain.linear(x, t[name].T).reshape(count, HEADS, HEAD_DIM)

    def routed(x):
        logits = plain.linear(x, t["b0.experts.router"].T).astype(np.float64)
        probabilities = np.exp(logits - logits.max(axis=-1, keepdims=True))
        probabilities /= probabilities.sum(axis=-1, keepdims=True)
        out = np.zeros_like(x)
        for row in range(count):
            e = int(np.argmax(probabilities[row]))
            one = x[row:row + 1]
            inner = plain.swiglu(plain.linear(one, t[f"b0.experts.{e}.gate"].T),
                                 plain.linear(one, t[f"b0.experts.{e}.up"].T))
            out[row] = plain.linear(inner, t[f"b0.experts.{e}.down"].T)[0] * probabilities[row, e]
        return out

    for block in (0, 1, 0):
        normed = plain.rms_norm(hidden, t[f"b{block}.norm1"], 1e-5)
        q, k, v = (heads_of(normed, f"b{block}.{name}") for name in ("q", "k", "v"))
        if block == 0:
            bias = t["b0.positions"][:count, None, :]
            q, k, window = q + bias, k + bias, None
        else:
            q, k, window = plain.rope_adjacent(q, cosine, sine), plain.rope_adjacent(k, cosine, sine), WINDOW
        context = plain.causal_attention(q.transpose(1, 0, 2), k.transpose(1, 0, 2),
                                         v.transpose(1, 0, 2), window=window)
        hidden = hidden + plain.linear(context.transpose(1, 0, 2).reshape(count, -1),
                                       t[f"b{block}.o"].T)
        normed = plain.rms_norm(hidden, t[f"b{block}.norm2"], 1e-5)
        if block == 0:
            hidden = (hidden + routed(normed)).astype(np.float32)
        else:
            inner = plain.swiglu(plain.linear(normed, t["b1.gate"].T), plain.linear(normed, t["b1.up"].T))
            hidden = (hidden + plain.linear(inner, t["b1.down"].T)).astype(np.float32)
    return plain.linear(plain.rms_norm(hidden, t["norm"], 1e-5), t["head"].T)


def test_routing_a_learned_position_encoding_and_a_window_step_like_their_plain_form(tmp_path):
    folder = str(tmp_path / "toy_routed")
    write_random_model(folder, ToyRoutedConfig(), seed=5, std=0.15, scale_std=0.3,
                       storage_dtype="float32")
    checkpoint = Checkpoint(folder)
    tensors = {name: checkpoint.read(name) for name in checkpoint.names()}
    harness = Harness(folder, "float32", page_size=4, num_pages=30, max_requests=3, max_tokens=64)
    kv_needs, state_needs = harness.model.cache_needs()
    assert sorted(kv_needs) == [0, 1, 2] and not state_needs
    # full attention (entries 0 and 2) and windowed attention (entry 1) have pages of their own
    assert sorted(len(group.entries) for group in harness.cache.groups) == [1, 2]

    a = random_tokens(VOCAB, 37, seed=11)
    b = random_tokens(VOCAB, 19, seed=12)
    expected_a, expected_b = plain_toy(tensors, a), plain_toy(tensors, b)
    # every expert is used by some token, or the routing shows nothing
    router = tensors["b0.experts.router"].float().numpy()
    tol = dict(atol=1e-4, rtol=2e-4)
    assert_close(harness.whole("a", a), expected_a, "whole a", **tol)
    out = harness.run([("a", a[:9], range(9)), ("b", b[:2], range(2))])
    assert_close(out, np.concatenate([expected_a[:9], expected_b[:2]]), "first portions", **tol)
    out = harness.run([("b", b[2:15], range(13)), ("a", a[9:11], range(2))])
    assert_close(out, np.concatenate([expected_b[2:15], expected_a[9:11]]), "second portions", **tol)
    for position in range(11, 37):
        step = [("a", [a[position]], [0])]
        other = 15 + position - 11
        if other < 19:
            step.append(("b", [b[other]], [0]))
        out = harness.run(step)
        assert_close(out[:1], expected_a[position:position + 1], f"a decode {position}", **tol)
        if len(step) == 2:
            assert_close(out[1:], expected_b[other:other + 1], f"b decode {other}", **tol)
    # the window gave pages back while a grew; the full group did not
    windowed = next(group for group in harness.cache.groups if group.need.window is not None)
    full = next(group for group in harness.cache.groups if group.need.window is None)
    assert windowed.pool.pages_in_use < full.pool.pages_in_use
    harness.end("a")
    harness.end("b")
    harness.cache.check()
    del router


def test_the_next_turn_of_a_conversation_adopts_its_prefix_across_a_windowed_group(tmp_path):
    """Prefix sharing with two cache groups, one of them windowed: the second prompt goes on
    from the first prompt and its answer, finds the first prompt's aligned prefix in the index
    and adopts it (every page of the full group, the window's last pages of the windowed one;
    free pages are poisoned, so a key read from a page the window gave back would show).
    Same tokens as an engine without the index, and as the plain form."""
    from helix_runtime_b200 import Engine
    folder = str(tmp_path / "toy_routed")
    write_random_model(folder, ToyRoutedConfig(), seed=5, std=0.15, scale_std=0.3,
                       storage_dtype="float32")
    checkpoint = Checkpoint(folder)
    tensors = {name: checkpoint.read(name) for name in checkpoint.names()}

    def conversation(engine):
        first = random_tokens(VOCAB, 18, seed=21)
        one = engine.generate([first], max_new_tokens=5)[0]
        second = first + one.generated_tokens + random_tokens(VOCAB, 6, seed=22)
        two = engine.generate([second], max_new_tokens=5)[0]
        return second, one, two

    options = dict(dtype="float32", page_size=4, num_pages=30, max_running_requests=2,
                   max_tokens_per_iteration=64, poison_free_pages=True)
    # the windowed layers get a pool of their own size: a window of 6 and pages of 4 are four
    # pages a request with a page of slack, times two requests, and two for the kept prefixes
    sharing = Engine.from_pretrained(folder, prefix_cache_entries=4, window_pages={WINDOW: 12},
                                     **options)
    assert sorted(group.pool.num_pages for group in sharing.cache.groups) == [12, 30]
    alone = Engine.from_pretrained(folder, **options)
    assert not sharing.model.graph_safe and sharing.graphs is None      # the routed part's word
    second, one, two = conversation(sharing)
    _, one_alone, two_alone = conversation(alone)
    assert one.generated_tokens == one_alone.generated_tokens
    assert two.generated_tokens == two_alone.generated_tokens
    logits = plain_toy(tensors, second + two.generated_tokens[:-1])
    for index, token in enumerate(two.generated_tokens):
        row = logits[len(second) + index - 1]
        assert row[token] >= row.max() - 1e-4, f"token {index}"
    stats = sharing.stats()["prefix"]
    assert stats["hits"] == 1 and stats["reused_tokens"] == 16 and stats["not_kept"] == 0
    assert sharing.request(two.request_id).reused_tokens == 16
    assert alone.request(two_alone.request_id).reused_tokens == 0
    sharing.cache.check()
    sharing.prefix.clear()
    sharing.cache.check()
    assert all(group.pool.pages_in_use == 0 for group in sharing.cache.groups)
