"""Each part of a layer alone, built from its spec at sizes other than the models', against
the plain functions: norm, attention (with its position encoding, grouped heads, a window, and
the checkpoint's half-split row order), feed-forward, embedding, head, and a block made of
them."""
from __future__ import annotations

import types

import numpy as np
import pytest
import torch

import plain_llama as plain
from engine_harness import assert_close
from helix_runtime_b200.cache import CacheManager
from helix_runtime_b200.config import BlockSpec, PartSpec
from helix_runtime_b200.engine.step import StepEntry, StepFunction
from helix_runtime_b200.models.decoder import Block
from helix_runtime_b200.parts import LayerCache, build_part

pytestmark = pytest.mark.gpu

DEVICE = torch.device("cuda:0")
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": dict(atol=2e-5, rtol=1e-4), "bfloat16": dict(atol=4e-2, rtol=4e-2)}


def scaled_tolerance(dtype, increment):
    """These tests feed unit-variance data through 0.2-variance weights, so outputs are tens of
    times larger than a model's; the plain functions here do not round intermediates.  For
    bfloat16 (8 significant bits per stored activation) allow 1 % of the output's own scale."""
    if dtype == "float32":
        scale = max(1.0, float(np.abs(increment).max()))
        return dict(atol=2e-5 * scale, rtol=1e-4)
    return dict(atol=0.01 * float(np.abs(increment).max()), rtol=2e-2)


def context_for(dtype, kv_needs, entries, page_size=8, num_pages=32, max_positions=128):
    """A step context for hand-made entries ``[(request, n_tokens)]`` (tokens do not matter)."""
    stub = types.SimpleNamespace(device=DEVICE, dtype=dtype, vocab_size=1 << 20,
                                 max_positions=max_positions)
    cache = CacheManager(kv_needs, {}, page_size, num_pages, 4, max_positions, dtype, DEVICE,
                         poison=True)
    step = StepFunction(stub, cache, max_tokens=256, max_requests=4, attention_split_keys=32)
    batch = []
    for request, count in entries:
        if not cache.has(request):
            cache.admit(request)
        batch.append(StepEntry(request, [0] * count, []))
    ctx, _, _, lengths = step.prepare(batch)
    return ctx, cache, step, batch, lengths


def held(array, dtype):
    return torch.as_tensor(np.asarray(array, dtype=np.float32)).to(DEVICE, dtype)


def as_numpy(tensor):
    return tensor.detach().float().cpu().numpy()


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    rng = np.random.default_rng(0)
    hidden = 200
    part = build_part("norm", PartSpec("rms", {"eps": 3e-4}, {"weight": "w"}), hidden)
    assert [(r.name, r.shape, r.role) for r in part.tensor_requests()] == [("w", (200,), "scale")]
    weight = (1 + 0.2 * rng.normal(size=hidden)).astype(np.float32)
    part.bind({"w": torch.as_tensor(weight)}, DTYPES[dtype], DEVICE)
    ctx, *_ = context_for(DTYPES[dtype], {}, [("a", 7)])
    x = (rng.normal(size=(7, hidden)) * 2).astype(np.float32)
    out = torch.empty((7, hidden), dtype=DTYPES[dtype], device=DEVICE)
    part.forward(ctx, held(x, torch.float32), out)
    assert_close(as_numpy(out), plain.rms_norm(x, weight, 3e-4), "rms norm", **TOL[dtype])


def attention_reference(x, w, heads, kv_heads, head_dim, theta, contexts, lengths, window, pairing):
    """Plain attention block on several requests, each alone: returns the residual increment."""
    outputs = []
    cursor = 0
    rotate = plain.rope_adjacent if pairing == "adjacent" else plain.rope_half_split
    for context, length in zip(contexts, lengths):
        rows = x[cursor:cursor + context + length]          # the request's whole history
        cursor += context + length
        count = rows.shape[0]
        cosine, sine = plain.rope_table(count, head_dim, theta)
        q = plain.linear(rows, w["q"].T).reshape(count, heads, head_dim)
        k = plain.linear(rows, w["k"].T).reshape(count, kv_heads, head_dim)
        v = plain.linear(rows, w["v"].T).reshape(count, kv_heads, head_dim)
        q = rotate(q, cosine, sine).transpose(1, 0, 2)
        k = rotate(k, cosine, sine).transpose(1, 0, 2)
        merged = plain.causal_attention(q, k, v.transpose(1, 0, 2), window=window)
        merged = merged.transpose(1, 0, 2).reshape(count, heads * head_dim)
        outputs.append(plain.linear(merged, w["o"].T)[context:])
    return np.concatenate(outputs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,window,checkpoint_pairing", [
    (6, 6, 16, None, "adjacent"), (6, 2, 16, None, "half_split"), (4, 4, 24, 5, "adjacent"),
    (3, 1, 64, None, "half_split"), (2, 2, 100, None, "half_split"), (4, 2, 6, None, "adjacent"),
    (2, 1, 144, None, "adjacent")])
def test_attention_part(dtype, heads, kv_heads, head_dim, window, checkpoint_pairing):
    rng = np.random.default_rng(1)
    hidden, theta = 96, 777.0
    position = PartSpec("rotary", {"theta": theta, "head_dim": head_dim, "rotary_dim": head_dim,
                                   "pairing": "adjacent", "max_positions": 128})
    spec = PartSpec("paged_attention",
                    {"num_heads": heads, "num_kv_heads": kv_heads, "head_dim": head_dim,
                     "scale": None, "window": window, "position": position,
                     "checkpoint_pairing": checkpoint_pairing},
                    {"q": "wq", "k": "wk", "v": "wv", "o": "wo"})
    part = build_part("mixer", spec, hidden)
    shapes = {r.name: r.shape for r in part.tensor_requests()}
    assert shapes == {"wq": (heads * head_dim, hidden), "wk": (kv_heads * head_dim, hidden),
                      "wv": (kv_heads * head_dim, hidden), "wo": (hidden, heads * head_dim)}
    need = part.kv_need()
    # a head that is no multiple of 16 is held in rows of the next multiple (zeros behind it)
    step = 16 if head_dim <= 128 else 32
    assert (need.kv_heads, need.head_dim, need.window) == (kv_heads, -(-head_dim // step) * step, window)
    weights = {name: as_numpy(held(rng.normal(size=shape) * 0.2, DTYPES[dtype]))
               for name, shape in shapes.items()}
    part.bind({name: torch.as_tensor(value) for name, value in weights.items()}, DTYPES[dtype],
              DEVICE)

    # two requests: the first is fed in two steps (a portion, then the rest), the second whole
    contexts, lengths = [11, 0], [9, 21]
    x_all = as_numpy(held(rng.normal(size=(sum(contexts) + sum(lengths), hidden)), DTYPES[dtype]))
    ctx, cache, step, batch, new_lengths = context_for(DTYPES[dtype], {0: need}, [("a", 11)])
    view = LayerCache(entry=0, owns=True, block_tables=cache.groups[0].device_tables,
                      page_size=8, num_pages=32, window=window)
    view.keys, view.values = cache.layer_storage(0)
    residual = torch.zeros((256, hidden), dtype=torch.float32, device=DEVICE)
    x = torch.zeros((256, hidden), dtype=DTYPES[dtype], device=DEVICE)
    x[:11] = held(x_all[:11], DTYPES[dtype])
    part.forward(ctx, view, x, residual)                    # fills the cache for request a
    step.finish(batch, new_lengths, ctx)

    batch = [StepEntry("a", [0] * 9, []), StepEntry("b", [0] * 21, [])]
    cache.admit("b")
    ctx, _, _, new_lengths = step.prepare(batch)
    x[:9] = held(x_all[11:20], DTYPES[dtype])
    x[9:30] = held(x_all[20:41], DTYPES[dtype])
    base = rng.normal(size=(30, hidden)).astype(np.float32)
    residual[:30] = held(base, torch.float32)
    part.forward(ctx, view, x, residual)
    step.raise_on_status()
    step.finish(batch, new_lengths, ctx)

    pairing = "adjacent" if checkpoint_pairing == "adjacent" else "half_split"
    w = {"q": weights["wq"], "k": weights["wk"], "v": weights["wv"], "o": weights["wo"]}
    expected = attention_reference(x_all, w, heads, kv_heads, head_dim, theta, contexts, lengths,
                                   window, pairing)
    assert_close(as_numpy(residual[:30]), base + expected, "attention part",
                 **scaled_tolerance(dtype, expected))
    cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,intermediate,tokens", [(96, 200, 13), (72, 44, 3), (128, 384, 70)])
def test_feed_forward_part(dtype, hidden, intermediate, tokens):
    rng = np.random.default_rng(2)
    spec = PartSpec("gated_mlp", {"intermediate_size": intermediate, "activation": "silu"},
                    {"gate": "g", "up": "u", "down": "d"})
    part = build_part("feed_forward", spec, hidden)
    shapes = {r.name: r.shape for r in part.tensor_requests()}
    assert shapes == {"g": (intermediate, hidden), "u": (intermediate, hidden),
                      "d": (hidden, intermediate)}
    weights = {name: as_numpy(held(rng.normal(size=shape) * 0.2, DTYPES[dtype]))
               for name, shape in shapes.items()}
    part.bind({name: torch.as_tensor(value) for name, value in weights.items()}, DTYPES[dtype],
              DEVICE)
    ctx, *_ = context_for(DTYPES[dtype], {}, [("a", tokens)])
    x = as_numpy(held(rng.normal(size=(tokens, hidden)), DTYPES[dtype]))
    base = rng.normal(size=(tokens, hidden)).astype(np.float32)
    residual = torch.zeros((256, hidden), dtype=torch.float32, device=DEVICE)
    residual[:tokens] = held(base, torch.float32)
    buffer = torch.zeros((256, hidden), dtype=DTYPES[dtype], device=DEVICE)
    buffer[:tokens] = held(x, DTYPES[dtype])
    part.forward(ctx, buffer, residual)
    expected = plain.linear(plain.swiglu(plain.linear(x, weights["g"].T),
                                         plain.linear(x, weights["u"].T)), weights["d"].T)
    assert_close(as_numpy(residual[:tokens]), base + expected, "feed-forward part",
                 **scaled_tolerance(dtype, expected))
    with pytest.raises(ValueError, match="silu"):
        build_part("feed_forward", PartSpec("gated_mlp", {"intermediate_size": 8,
                                                          "activation": "gelu"}, spec.tensors), 8)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    rng = np.random.default_rng(3)
    hidden, vocab = 88, 301
    table = as_numpy(held(rng.normal(size=(vocab, hidden)), DTYPES[dtype]))
    head_weight = as_numpy(held(rng.normal(size=(vocab, hidden)) * 0.1, DTYPES[dtype]))
    embedding = build_part("embedding", PartSpec("token_table", {"vocab_size": vocab},
                                                 {"weight": "e"}), hidden)
    head = build_part("lm_head", PartSpec("linear", {"vocab_size": vocab, "tied": False},
                                          {"weight": "h"}), hidden)
    embedding.bind({"e": torch.as_tensor(table)}, DTYPES[dtype], DEVICE)
    head.bind({"h": torch.as_tensor(head_weight)}, DTYPES[dtype], DEVICE)
    ctx, *_ = context_for(DTYPES[dtype], {}, [("a", 5)])
    ids = [300, 0, 17, 17, 123]
    ctx.token_ids[:5] = torch.tensor(ids, dtype=torch.int32, device=DEVICE)
    residual = torch.zeros((256, hidden), dtype=torch.float32, device=DEVICE)
    embedding.forward(ctx, residual)
    np.testing.assert_array_equal(as_numpy(residual[:5]), table[ids])
    x = as_numpy(held(rng.normal(size=(5, hidden)), DTYPES[dtype]))
    buffer = torch.zeros((256, hidden), dtype=DTYPES[dtype], device=DEVICE)
    buffer[:5] = held(x, DTYPES[dtype])
    logits = torch.zeros((256, vocab), dtype=torch.float32, device=DEVICE)
    head.forward(ctx, buffer, logits, 5)
    assert_close(as_numpy(logits[:5]), plain.linear(x, head_weight.T), "head",
                 atol=2e-4, rtol=1e-4)


def test_block_wires_its_parts_in_pre_norm_order():
    rng = np.random.default_rng(4)
    hidden, heads, head_dim, inter = 64, 4, 16, 104
    position = PartSpec("rotary", {"theta": 10000.0, "head_dim": head_dim, "rotary_dim": head_dim,
                                   "pairing": "adjacent", "max_positions": 128})
    spec = BlockSpec(
        arrangement="pre_norm",
        mixer_norm=PartSpec("rms", {"eps": 1e-5}, {"weight": "n1"}),
        mixer=PartSpec("paged_attention", {"num_heads": heads, "num_kv_heads": heads,
                                           "head_dim": head_dim, "scale": None, "window": None,
                                           "position": position, "checkpoint_pairing": "adjacent"},
                       {"q": "q", "k": "k", "v": "v", "o": "o"}),
        feed_forward_norm=PartSpec("rms", {"eps": 1e-5}, {"weight": "n2"}),
        feed_forward=PartSpec("gated_mlp", {"intermediate_size": inter, "activation": "silu"},
                              {"gate": "g", "up": "u", "down": "d"}))
    block = Block(spec, hidden)
    tensors = {}
    for part in block.parts():
        for request in part.tensor_requests():
            value = 1 + 0.1 * rng.normal(size=request.shape) if request.role == "scale" \
                else 0.15 * rng.normal(size=request.shape)
            tensors[request.name] = torch.as_tensor(value.astype(np.float32))
        part.bind(tensors, torch.float32, DEVICE)
    w = {name: value.numpy() for name, value in tensors.items()}
    tokens = 19
    ctx, cache, step, batch, lengths = context_for(torch.float32, {0: block.mixer.kv_need()},
                                                   [("a", tokens)])
    view = LayerCache(entry=0, owns=True, block_tables=cache.groups[0].device_tables, page_size=8,
                      num_pages=32)
    view.keys, view.values = cache.layer_storage(0)
    x = rng.normal(size=(tokens, hidden)).astype(np.float32)
    residual = torch.zeros((256, hidden), dtype=torch.float32, device=DEVICE)
    residual[:tokens] = held(x, torch.float32)
    normed = torch.zeros((256, hidden), dtype=torch.float32, device=DEVICE)
    block.forward(ctx, view, residual, normed)
    step.raise_on_status()

    normed1 = plain.rms_norm(x, w["n1"], 1e-5)
    attention = attention_reference(normed1, {"q": w["q"], "k": w["k"], "v": w["v"], "o": w["o"]},
                                    heads, heads, head_dim, 10000.0, [0], [tokens], None, "adjacent")
    after_attention = (x + attention).astype(np.float32)
    normed2 = plain.rms_norm(after_attention, w["n2"], 1e-5)
    mlp = plain.linear(plain.swiglu(plain.linear(normed2, w["g"].T), plain.linear(normed2, w["u"].T)),
                       w["d"].T)
    assert_close(as_numpy(residual[:tokens]), after_attention + mlp, "block", atol=2e-5, rtol=1e-4)
    with pytest.raises(ValueError, match="arrangement"):
        Block(BlockSpec("post_norm", spec.mixer_norm, spec.mixer, spec.feed_forward_norm,
                        spec.feed_forward), hidden)
