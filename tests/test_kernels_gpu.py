"""Each CUDA kernel alone against its plain reference, at sizes other than the engine's.

References are the NumPy functions of ``plain_llama`` (double accumulators) or a few lines of
NumPy written here from the same formulas.
"""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_llama as plain
from engine_harness import assert_close
from helix_runtime_b200.ops import library as ops

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def dev(array, dtype=torch.float32):
    return torch.as_tensor(np.asarray(array)).to(device=DEVICE, dtype=dtype).contiguous()


def host(tensor):
    return tensor.detach().float().cpu().numpy()


def status_word():
    return torch.zeros(1, dtype=torch.int32, device=DEVICE)


def cache_chunk(dtype, head_dim):
    """Elements per 16-byte chunk of the cache layout (the widest of 16 bytes, 4 or 2 elements
    that divides the head size)."""
    widest = 8 if dtype == torch.bfloat16 else 4
    for chunk in (widest, 4, 2):
        if chunk <= widest and head_dim % chunk == 0:
            return chunk
    raise ValueError(head_dim)


def to_cache_layout(keys, dtype):
    """[page, kv_head, slot, dim] -> the cache's [page, kv_head, dim / chunk, slot, chunk]
    (kept in an array of the same shape)."""
    pages, heads, slots, dim = keys.shape
    c = cache_chunk(dtype, dim)
    return keys.reshape(pages, heads, slots, dim // c, c).transpose(0, 1, 3, 2, 4).reshape(keys.shape)


def from_cache_layout(cache, dtype):
    pages, heads, slots, dim = cache.shape
    c = cache_chunk(dtype, dim)
    return cache.reshape(pages, heads, dim // c, slots, c).transpose(0, 1, 3, 2, 4).reshape(cache.shape)


def rounded(array, dtype):
    """The values a tensor of ``dtype`` actually holds, as float32."""
    return host(dev(array, dtype))


# ------------------------------------------------------------------- embedding

@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_gathers_rows_and_flags_bad_ids(dtype):
    rng = np.random.default_rng(0)
    vocab, hidden = 1000, 72
    table = dev(rng.normal(size=(vocab, hidden)), dtype)
    ids = torch.tensor([0, 999, 17, 17, 500], dtype=torch.int32, device=DEVICE)
    out = torch.empty((5, hidden), dtype=torch.float32, device=DEVICE)
    status = status_word()
    ops.embed(table, ids, out, status)
    np.testing.assert_array_equal(host(out), host(table)[[0, 999, 17, 17, 500]])
    assert int(status.item()) == 0
    bad = torch.tensor([3, 1000, -1], dtype=torch.int32, device=DEVICE)
    out = torch.zeros((3, hidden), dtype=torch.float32, device=DEVICE)
    ops.embed(table, bad, out, status)
    result = host(out)
    np.testing.assert_array_equal(result[0], host(table)[3])
    assert np.isnan(result[1]).all() and np.isnan(result[2]).all()
    assert int(status.item()) & ops.FLAG_BAD_TOKEN


# --------------------------------------------------------------------- RMSNorm

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,eps", [(200, 1e-5), (4104, 1e-6), (24, 1e-3), (4096, 1e-5),
                                        (5120, 1e-5), (8192, 1e-6), (8200, 1e-5), (1022, 1e-5)])
def test_rmsnorm(dtype, hidden, eps):
    rng = np.random.default_rng(1)
    x = (rng.normal(size=(7, hidden)) * 3.0).astype(np.float32)
    w = (1.0 + 0.3 * rng.normal(size=hidden)).astype(np.float32)
    out = torch.empty((7, hidden), dtype=dtype, device=DEVICE)
    ops.rmsnorm(dev(x), dev(w), out, eps)
    expected = plain.rms_norm(x, w, eps)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=1e-2, rtol=8e-3)
    assert_close(host(out), expected, "rmsnorm", **tol)
    # gathered rows (the final norm runs on the wanted rows only)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEVICE)
    out = torch.empty((3, hidden), dtype=dtype, device=DEVICE)
    ops.rmsnorm(dev(x), dev(w), out, eps, rows)
    assert_close(host(out), expected[[6, 0, 3]], "rmsnorm gathered", **tol)


# ---------------------------------------------------------------------- SwiGLU

@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    rng = np.random.default_rng(2)
    tokens, inter = 9, 176
    gate_up = (rng.normal(size=(tokens, 2 * inter)) * 4.0).astype(np.float32)
    gate_up[0, :4] = [-100.0, 100.0, 0.0, -20.0]
    act = torch.empty((tokens, inter), dtype=dtype, device=DEVICE)
    ops.swiglu(dev(gate_up), act)
    expected = plain.swiglu(gate_up[:, :inter], gate_up[:, inter:])
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=1e-2, rtol=8e-3)
    assert_close(host(act), expected, "swiglu", **tol)


def test_swiglu_clears_a_split_k_accumulator():
    rng = np.random.default_rng(21)
    gate_up = (rng.normal(size=(5, 2 * 88)) * 3.0).astype(np.float32)
    buffer = dev(gate_up)
    act = torch.empty((5, 88), dtype=torch.bfloat16, device=DEVICE)
    ops.swiglu(buffer, act, zero_input=True)
    assert_close(host(act), plain.swiglu(gate_up[:, :88], gate_up[:, 88:]), "swiglu",
                 atol=1e-2, rtol=8e-3)
    assert float(buffer.abs().sum()) == 0.0


# -------------------------------------------------------------- matrix products

def product_reference(x, w):
    return (x.astype(np.float64) @ w.astype(np.float64).T).astype(np.float32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,features,depth", [(37, 83, 45), (1, 130, 257), (130, 64, 64)])
def test_gemm_on_cuda_cores(dtype, tokens, features, depth):
    rng = np.random.default_rng(3)
    x = rounded(rng.normal(size=(tokens, depth)), dtype)
    w = rounded(rng.normal(size=(features, depth)) * 0.1, dtype)
    expected = product_reference(x, w)
    tight = dict(atol=2e-5, rtol=2e-5)
    out = torch.empty((tokens, features), dtype=dtype, device=DEVICE)
    ops.gemm_simt(dev(x, dtype), dev(w, dtype), out, tokens, ops.EPI_STORE)
    assert_close(host(out), expected, "store",
                 **(tight if dtype == torch.float32 else dict(atol=2e-2, rtol=8e-3)))
    out32 = torch.empty((tokens, features), dtype=torch.float32, device=DEVICE)
    ops.gemm_simt(dev(x, dtype), dev(w, dtype), out32, tokens, ops.EPI_STORE_F32)
    assert_close(host(out32), expected, "store f32", **tight)
    base = rng.normal(size=(tokens, features)).astype(np.float32)
    acc = dev(base)
    ops.gemm_simt(dev(x, dtype), dev(w, dtype), acc, tokens, ops.EPI_ADD_F32)
    assert_close(host(acc), base + expected, "add f32", **tight)


TC_SHAPES = [
    # tokens, features, depth: every token tile (16..256), ragged edges in all three sizes
    (1, 64, 64), (5, 200, 120), (16, 384, 328), (17, 128, 1024), (40, 136, 72),
    (100, 256, 4096), (130, 384, 200), (300, 520, 328), (513, 128, 64),
    # more tiles than SMs: CTAs of the persistent kernel take three tiles and more, so both
    # accumulators in tensor memory are used again
    (1100, 9000, 136),
    # the add epilogue shares a short last round out by k-blocks: 45 tiles of 64 k-blocks for
    # the whole grid (every tile in pieces, ragged edges in tokens and features), and 188 tiles
    # on 148 SMs (one round of whole tiles, then 40 tiles in pieces)
    (600, 2250, 4096), (512, 12032, 4096),
]


@pytest.mark.parametrize("tiled", [False, True])
@pytest.mark.parametrize("tokens,features,depth", TC_SHAPES)
def test_gemm_on_tensor_cores(tokens, features, depth, tiled):
    """``tiled``: the weights are handed over as [128 x 64] tiles (how the engine stores the
    matrices of its tensor-core products), zero padded in both directions."""
    rng = np.random.default_rng(4)
    x = rounded(rng.normal(size=(tokens, depth)), torch.bfloat16)
    w = rounded(rng.normal(size=(features, depth)) * 0.1, torch.bfloat16)
    expected = product_reference(x, w)
    status = status_word()
    xd, wd = dev(x, torch.bfloat16), dev(w, torch.bfloat16)
    if tiled:
        tiles = ops.tile_weights(wd)
        assert tiles.shape == (-(-features // 128), -(-depth // 64), 128, 64)
        row_major = ops.gemm_tc

        def gemm_tc(x_, w_, *args, **kwargs):
            return row_major(x_, tiles, *args, weight_shape=(features, depth), **kwargs)
    else:
        gemm_tc = ops.gemm_tc
    assert ops.gemm_tc_supports(tokens, features, depth, depth, depth)
    tight = dict(atol=1e-4 * math.sqrt(depth / 64), rtol=2e-5)

    out32 = torch.full((tokens, features), float("nan"), dtype=torch.float32, device=DEVICE)
    gemm_tc(xd, wd, out32, tokens, features, ops.EPI_STORE_F32, status)
    assert_close(host(out32), expected, "store f32", **tight)

    out16 = torch.full((tokens, features), float("nan"), dtype=torch.bfloat16, device=DEVICE)
    gemm_tc(xd, wd, out16, tokens, features, ops.EPI_STORE, status)
    assert_close(host(out16), expected, "store bf16", atol=2e-2, rtol=8e-3)

    base = rng.normal(size=(tokens, features)).astype(np.float32)
    for splits in (1, 3):
        acc = dev(base)
        gemm_tc(xd, wd, acc, tokens, features, ops.EPI_ADD_F32, status, k_splits=splits)
        assert_close(host(acc), base + expected, f"add f32 with {splits} k-splits", **tight)
    assert int(status.item()) == 0


@pytest.mark.parametrize("tokens,inter,depth", [(3, 176, 64), (33, 320, 120), (200, 1000, 264),
                                                 (64, 128, 512), (1100, 4600, 72),
                                                 (300, 1024, 200), (20, 256, 72)])
def test_gemm_with_swiglu_epilogue(tokens, inter, depth):
    rng = np.random.default_rng(5)
    x = rounded(rng.normal(size=(tokens, depth)), torch.bfloat16)
    w = rounded(rng.normal(size=(2 * inter, depth)) * 0.2, torch.bfloat16)
    gate = product_reference(x, w[:inter])
    up = product_reference(x, w[inter:])
    expected = plain.swiglu(gate, up)
    status = status_word()
    act = torch.full((tokens, inter), float("nan"), dtype=torch.bfloat16, device=DEVICE)
    ops.gemm_tc(dev(x, torch.bfloat16), dev(w, torch.bfloat16), act, tokens, inter,
                ops.EPI_SWIGLU, status, up_row_offset=inter)
    assert_close(host(act), expected, "swiglu epilogue", atol=2e-2, rtol=8e-3)
    if inter % 128 == 0:       # up rows begin on a tile: the same from tiled weights
        act.fill_(float("nan"))
        ops.gemm_tc(dev(x, torch.bfloat16), ops.tile_weights(dev(w, torch.bfloat16)), act, tokens,
                    inter, ops.EPI_SWIGLU, status, up_row_offset=inter,
                    weight_shape=(2 * inter, depth))
        assert_close(host(act), expected, "swiglu epilogue, tiled weights", atol=2e-2, rtol=8e-3)
    else:
        with pytest.raises(ops.KernelError, match="multiple of 128"):
            ops.gemm_tc(dev(x, torch.bfloat16), ops.tile_weights(dev(w, torch.bfloat16)), act,
                        tokens, inter, ops.EPI_SWIGLU, status, up_row_offset=inter,
                        weight_shape=(2 * inter, depth))
    assert int(status.item()) == 0


def test_tensor_core_gemm_refuses_depths_it_cannot_load():
    x = torch.zeros((4, 44), dtype=torch.bfloat16, device=DEVICE)
    w = torch.zeros((8, 44), dtype=torch.bfloat16, device=DEVICE)
    out = torch.zeros((4, 8), dtype=torch.float32, device=DEVICE)
    assert not ops.gemm_tc_supports(4, 8, 44, 44, 44)
    with pytest.raises(ops.KernelError, match="not supported"):
        ops.gemm_tc(x, w, out, 4, 8, ops.EPI_STORE_F32, status_word())


# ------------------------------------------------- rotary encoding + cache append

def rope_reference(x, positions, theta, rotary_dim, pairing):
    """x [T, heads, D]; the plain rotation applied to the first ``rotary_dim`` coordinates."""
    out = x.copy()
    for t, position in enumerate(positions):
        cosine, sine = plain.rope_table(1, rotary_dim, theta, offset=int(position))
        part = x[t:t + 1, :, :rotary_dim]
        rotate = plain.rope_adjacent if pairing == "adjacent" else plain.rope_half_split
        out[t:t + 1, :, :rotary_dim] = rotate(part, cosine, sine)
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,rotary_dim,pairing", [
    (4, 4, 16, 16, "adjacent"), (6, 2, 24, 24, "half_split"), (3, 1, 32, 16, "adjacent"),
    (5, 5, 100, 100, "adjacent"), (2, 2, 48, 32, "half_split"),
    (12, 12, 128, 128, "adjacent"), (48, 8, 64, 64, "adjacent"), (20, 10, 96, 64, "adjacent"),
    # a rotary part that ends inside a 16-byte piece of the head (100 of 112, 20 of 40)
    (3, 1, 112, 100, "adjacent"), (2, 2, 40, 20, "adjacent")])
@pytest.mark.parametrize("long_portions", [False, True])
def test_rope_and_cache_append(dtype, heads, kv_heads, head_dim, rotary_dim, pairing, long_portions):
    rng = np.random.default_rng(6)
    theta, max_positions = 50000.0, 96
    if not long_portions:
        page_size, num_pages = 8, 12
        # two requests: one continues at position 13 (inside a page), one starts at 0
        positions = np.array([13, 14, 15, 16, 17, 0, 1, 2], dtype=np.int32)
        token_request = np.array([0, 0, 0, 0, 0, 1, 1, 1], dtype=np.int32)
        slots = np.array([2, 0], dtype=np.int32)
        tables = np.full((3, 12), -1, dtype=np.int32)
        tables[2, :3] = [7, 3, 9]
        tables[0, :1] = [5]
    else:
        # portions of 37 and 21 tokens over several pages: one continues at position 13,
        # inside a page
        page_size, num_pages = 16, 12
        positions = np.array(list(range(13, 50)) + list(range(0, 21)), dtype=np.int32)
        token_request = np.array([0] * 37 + [1] * 21, dtype=np.int32)
        slots = np.array([2, 0], dtype=np.int32)
        tables = np.full((3, 6), -1, dtype=np.int32)
        tables[2, :4] = [7, 3, 9, 1]
        tables[0, :2] = [5, 10]
    tokens = len(positions)
    width = (heads + 2 * kv_heads) * head_dim
    qkv = rounded(rng.normal(size=(tokens, width)), dtype)
    half = max(rotary_dim // 2, 1)
    exponent = -2.0 * np.arange(half) / rotary_dim
    angle = np.arange(max_positions)[:, None] * np.power(np.float64(np.float32(theta)), exponent)[None, :]
    cos, sin = dev(np.cos(angle)), dev(np.sin(angle))
    k_cache = torch.full((num_pages, kv_heads, page_size, head_dim), float("nan"), dtype=dtype, device=DEVICE)
    v_cache = torch.full_like(k_cache, float("nan"))
    buffer = dev(qkv, dtype)
    status = status_word()
    ops.rope_append(buffer, dev(positions, torch.int32), dev(token_request, torch.int32),
                    dev(slots, torch.int32), dev(tables, torch.int32), k_cache, v_cache, cos, sin,
                    tokens, heads, kv_heads, head_dim, rotary_dim,
                    {"adjacent": 0, "half_split": 1}[pairing], page_size, num_pages, status)
    assert int(status.item()) == 0
    q = qkv[:, :heads * head_dim].reshape(tokens, heads, head_dim)
    k = qkv[:, heads * head_dim:(heads + kv_heads) * head_dim].reshape(tokens, kv_heads, head_dim)
    v = qkv[:, (heads + kv_heads) * head_dim:].reshape(tokens, kv_heads, head_dim)
    q_expected = rope_reference(q, positions, theta, rotary_dim, pairing)
    k_expected = rope_reference(k, positions, theta, rotary_dim, pairing)
    tol = dict(atol=2e-6, rtol=2e-6) if dtype == torch.float32 else dict(atol=2e-2, rtol=8e-3)
    result = host(buffer)
    assert_close(result[:, :heads * head_dim].reshape(q.shape), q_expected, "rotated queries", **tol)
    np.testing.assert_array_equal(result[:, (heads + kv_heads) * head_dim:],
                                  qkv[:, (heads + kv_heads) * head_dim:])
    keys, values = from_cache_layout(host(k_cache), dtype), from_cache_layout(host(v_cache), dtype)
    written = np.zeros((num_pages, page_size), dtype=bool)
    for t in range(tokens):
        page = tables[slots[token_request[t]], positions[t] // page_size]
        slot = positions[t] % page_size
        written[page, slot] = True
        assert_close(keys[page, :, slot], k_expected[t], f"key of token {t}", **tol)
        np.testing.assert_array_equal(values[page, :, slot], v[t])
    # nothing else was touched
    untouched = ~written[:, None, :].repeat(kv_heads, axis=1)
    assert np.isnan(keys[untouched]).all() and np.isnan(values[untouched]).all()


def test_rope_reads_and_clears_a_split_k_accumulator():
    """The projection may arrive as float32 sums: the kernel must round them to bfloat16 as
    the projection's store would have, rotate, write the cache, and leave zeros behind."""
    rng = np.random.default_rng(22)
    heads, kv_heads, head_dim, page_size, num_pages = 3, 3, 32, 8, 4
    tokens = 4
    width = (heads + 2 * kv_heads) * head_dim
    sums = rng.normal(size=(8, width)).astype(np.float32)
    positions = np.array([5, 6, 7, 8], dtype=np.int32)
    tables = np.array([[2, 0, -1, -1]], dtype=np.int32)
    angle = np.arange(32)[:, None] * np.power(10000.0, -2.0 * np.arange(16) / 32)[None, :]
    cos, sin = dev(np.cos(angle)), dev(np.sin(angle))
    outputs = []
    for use_accumulator in (False, True):
        k_cache = torch.zeros((num_pages, kv_heads, page_size, head_dim), dtype=torch.bfloat16,
                              device=DEVICE)
        v_cache = torch.zeros_like(k_cache)
        qkv = dev(sums[:tokens], torch.bfloat16) if not use_accumulator else \
            torch.full((tokens, width), float("nan"), dtype=torch.bfloat16, device=DEVICE)
        accum = dev(sums) if use_accumulator else None
        ops.rope_append(qkv, dev(positions, torch.int32), dev(np.zeros(4), torch.int32),
                        dev(np.zeros(1), torch.int32), dev(tables, torch.int32), k_cache, v_cache,
                        cos, sin, tokens, heads, kv_heads, head_dim, head_dim, 0, page_size,
                        num_pages, status_word(), accum=accum)
        outputs.append((host(qkv)[:, :heads * head_dim], host(k_cache), host(v_cache)))
        if use_accumulator:
            cleared = host(accum)
            assert np.abs(cleared[:tokens]).sum() == 0.0
            np.testing.assert_array_equal(cleared[tokens:], sums[tokens:])   # other rows untouched
    for direct, through_accumulator in zip(*outputs):
        np.testing.assert_array_equal(direct, through_accumulator)


@pytest.mark.parametrize("dtype,head_dim", [(torch.float32, 24), (torch.bfloat16, 32)])
def test_rope_flags_a_position_beyond_its_table(dtype, head_dim):
    """A caller whose positions run past the cos/sin table gets the bad-position flag (the row
    is rotated with the table's last row: nothing outside the table is read)."""
    heads = kv_heads = 2
    page_size, num_pages, table_positions = 8, 4, 16
    width = (heads + 2 * kv_heads) * head_dim
    half = head_dim // 2
    angle = np.arange(table_positions)[:, None] * np.power(10000.0, -2.0 * np.arange(half) / head_dim)
    cos, sin = dev(np.cos(angle)), dev(np.sin(angle))
    tables = dev(np.array([[1, 3, 0, 2]]), torch.int32)
    zeros = dev(np.zeros(2), torch.int32)
    for positions, expected in (([14, 15], 0), ([15, 16], ops.FLAG_BAD_POSITION)):
        qkv = dev(np.random.default_rng(5).normal(size=(2, width)), dtype)
        k_cache = torch.zeros((num_pages, kv_heads, page_size, head_dim), dtype=dtype, device=DEVICE)
        status = status_word()
        ops.rope_append(qkv, dev(positions, torch.int32), zeros, zeros[:1], tables, k_cache,
                        torch.zeros_like(k_cache), cos, sin, 2, heads, kv_heads, head_dim,
                        head_dim, 0, page_size, num_pages, status)
        assert int(status.item()) == expected
        assert np.isfinite(host(qkv)).all()


@pytest.mark.parametrize("tiled", [False, True])
@pytest.mark.parametrize("heads,kv_heads,head_dim,rotary_dim,depth,page_size", [
    (4, 4, 16, 16, 64, 8), (3, 1, 112, 100, 200, 16), (6, 2, 64, 32, 264, 32),
    (5, 5, 128, 128, 128, 16)])
@pytest.mark.parametrize("own_cache", [True, False])
def test_product_with_rotary_append_epilogue(heads, kv_heads, head_dim, rotary_dim, depth,
                                             page_size, tiled, own_cache):
    """The fused QKV product of prompt portions against the plain product followed by the
    rotary/append kernel: rotated queries, and keys and values in their pages, must agree;
    rows of the output beyond the tokens and every other slot of the cache stay untouched."""
    rng = np.random.default_rng(31)
    # three requests in one step: one continues at position 13 (inside a page), one starts at
    # 0 and spans token tiles, one brings a single token; 301 tokens: the last tile is ragged
    counts, starts = [150, 150, 1], [13, 0, 77]
    positions = np.concatenate([np.arange(s, s + c) for s, c in zip(starts, counts)]).astype(np.int32)
    token_request = np.concatenate([[r] * c for r, c in enumerate(counts)]).astype(np.int32)
    tokens, max_positions = len(positions), 192
    slots = np.array([2, 0, 3], dtype=np.int32)
    per_request = -(-max_positions // page_size)
    num_pages = 3 * per_request + 2
    tables = np.full((4, per_request), -1, dtype=np.int32)
    order = rng.permutation(num_pages)
    for r in range(3):
        tables[slots[r]] = order[r * per_request:(r + 1) * per_request]
    width = (heads + 2 * kv_heads) * head_dim
    x = dev(rounded(rng.normal(size=(tokens + 5, depth)), torch.bfloat16), torch.bfloat16)
    w = dev(rounded(rng.normal(size=(width, depth)) / math.sqrt(depth), torch.bfloat16), torch.bfloat16)
    held = ops.tile_weights(w) if tiled else w
    half = max(rotary_dim // 2, 1)
    exponent = -2.0 * np.arange(half) / rotary_dim
    angle = np.arange(max_positions)[:, None] * np.power(10000.0, exponent)[None, :]
    cos, sin = dev(np.cos(angle)), dev(np.sin(angle))
    device_args = (dev(positions, torch.int32), dev(token_request, torch.int32),
                   dev(slots, torch.int32), dev(tables, torch.int32))

    def caches():
        k = torch.full((num_pages, kv_heads, page_size, head_dim), float("nan"),
                       dtype=torch.bfloat16, device=DEVICE)
        return (k, torch.full_like(k, float("nan"))) if own_cache else (None, None)

    # the two-kernel way
    qkv = torch.full((tokens + 5, width), float("nan"), dtype=torch.bfloat16, device=DEVICE)
    k_plain, v_plain = caches()
    status = status_word()
    ops.gemm_tc(x, held, qkv, tokens, width, ops.EPI_STORE, status, weight_shape=(width, depth))
    ops.rope_append(qkv, *device_args, k_plain, v_plain, cos, sin, tokens, heads, kv_heads,
                    head_dim, rotary_dim, 0, page_size, num_pages, status)
    # the fused way
    fused = torch.full((tokens + 5, width), float("nan"), dtype=torch.bfloat16, device=DEVICE)
    k_fused, v_fused = caches()
    ops.gemm_tc_rope_append(x, held, fused, tokens, device_args[0], device_args[1],
                            device_args[2], device_args[3] if own_cache else None, k_fused,
                            v_fused, cos, sin, heads, kv_heads, head_dim, rotary_dim, page_size,
                            num_pages, status, weight_shape=(width, depth))
    assert int(status.item()) == 0
    q_size = heads * head_dim
    plain_q, fused_q = host(qkv)[:tokens, :q_size], host(fused)[:tokens, :q_size]
    assert np.isfinite(fused_q).all()
    # the same products rounded the same way, then the same rotation: one bfloat16 step at most
    assert_close(fused_q, plain_q, "rotated queries", atol=1e-6, rtol=2.0 ** -7)
    assert np.isnan(host(fused)[tokens:]).all() and np.isnan(host(fused)[:, q_size:]).all()
    if own_cache:
        for name, one, other in (("keys", k_fused, k_plain), ("values", v_fused, v_plain)):
            one, other = host(one), host(other)
            np.testing.assert_array_equal(np.isnan(one), np.isnan(other))
            filled = ~np.isnan(other)
            assert filled.sum() == tokens * kv_heads * head_dim
            assert_close(one[filled], other[filled], name, atol=1e-6, rtol=2.0 ** -7)


def test_product_with_rotary_append_epilogue_refuses_short_portions_and_odd_heads():
    x = torch.zeros((128, 64), dtype=torch.bfloat16, device=DEVICE)
    w = torch.zeros((3 * 2 * 24, 64), dtype=torch.bfloat16, device=DEVICE)
    out = torch.zeros((128, 3 * 2 * 24), dtype=torch.bfloat16, device=DEVICE)
    ints = torch.zeros(128, dtype=torch.int32, device=DEVICE)
    table = torch.zeros((1, 4), dtype=torch.float32, device=DEVICE)
    with pytest.raises(ops.KernelError, match="multiple of 16"):
        ops.gemm_tc_rope_append(x, w, out, 128, ints, ints, ints, None, None, None, table, table,
                                2, 2, 24, 8, 16, 4, status_word())
    w = torch.zeros((3 * 2 * 32, 64), dtype=torch.bfloat16, device=DEVICE)
    out = torch.zeros((128, 3 * 2 * 32), dtype=torch.bfloat16, device=DEVICE)
    assert ops.gemm_tc_rope_append_min_tokens() == 65
    with pytest.raises(ops.KernelError, match="at least 65"):
        ops.gemm_tc_rope_append(x, w, out, 64, ints, ints, ints, None, None, None, table, table,
                                2, 2, 32, 8, 16, 4, status_word())


# ------------------------------------------------------------------- attention

def attention_case(rng, dtype, heads, kv_heads, head_dim, page_size, contexts, new_tokens,
                   window, split_keys, dominant=None, tensor_core_min=0, lost_page=None,
                   tensor_memory=None, max_splits=None):
    """Build a paged cache holding ``contexts[r] + new_tokens[r]`` keys per request in shuffled
    pages and the queries of the new tokens; return kernel output and plain reference.
    ``lost_page=(request, index)`` points that entry of the block table outside the pool: the
    kernel has to raise the bad-page flag and go on without those keys."""
    requests = len(contexts)
    totals = [c + n for c, n in zip(contexts, new_tokens)]
    pages_per = [-(-t // page_size) for t in totals]
    num_pages = sum(pages_per) + 3
    order = rng.permutation(num_pages)
    max_pages = max(pages_per) + 1
    tables = np.full((requests + 2, max_pages), -1, dtype=np.int32)
    slots = rng.permutation(requests + 2)[:requests].astype(np.int32)
    cursor = 0
    keys = [rounded(rng.normal(size=(kv_heads, t, head_dim)), dtype) for t in totals]
    values = [rounded(rng.normal(size=(kv_heads, t, head_dim)), dtype) for t in totals]
    queries = [rounded(rng.normal(size=(heads, n, head_dim)), dtype) for n in new_tokens]
    if dominant is not None:
        # make one far key win: its direction equals the query's, scaled up
        for r, key_position in dominant.items():
            for head in range(heads):
                kv = head // (heads // kv_heads)
                direction = queries[r][head, -1] / np.linalg.norm(queries[r][head, -1])
                keys[r][kv, key_position] = rounded(direction * 40.0, dtype)
    k_cache = np.full((num_pages, kv_heads, page_size, head_dim), np.nan, dtype=np.float32)
    v_cache = np.full_like(k_cache, np.nan)
    for r in range(requests):
        for p in range(pages_per[r]):
            page = order[cursor]
            cursor += 1
            tables[slots[r], p] = page
            lo, hi = p * page_size, min((p + 1) * page_size, totals[r])
            k_cache[page, :, :hi - lo] = keys[r][:, lo:hi]
            v_cache[page, :, :hi - lo] = values[r][:, lo:hi]
    lost_keys = None
    if lost_page is not None:
        r, p = lost_page
        tables[slots[r], p] = num_pages + 5
        lost_keys = (r, p * page_size, min((p + 1) * page_size, totals[r]))
    positions, token_request, q_rows = [], [], []
    for r in range(requests):
        for i in range(new_tokens[r]):
            positions.append(contexts[r] + i)
            token_request.append(r)
            q_rows.append(queries[r][:, i].reshape(-1))
    tokens = len(positions)
    q = np.stack(q_rows)
    scale = 1.0 / math.sqrt(head_dim)
    longest = max(totals) if not window else min(max(totals), window)
    max_splits = max_splits or max(1, -(-longest // split_keys))
    partial = None
    if max_splits > 1:
        partial = torch.empty(ops.attention_scratch_floats(tokens, heads, head_dim, max_splits),
                              dtype=torch.float32, device=DEVICE)
    out = torch.full((tokens, heads * head_dim), float("nan"), dtype=dtype, device=DEVICE)
    status = status_word()
    starts = dev(np.concatenate([[0], np.cumsum(new_tokens)]), torch.int32)
    if tensor_core_min:
        # requests with at least that many tokens on the tensor cores, the rest (if any) on
        # the CUDA cores: together they must fill every row
        ops.prefill_attention(dev(q, dtype), dev(to_cache_layout(k_cache, dtype), dtype),
                              dev(to_cache_layout(v_cache, dtype), dtype), starts,
                              dev(contexts, torch.int32), dev(slots, torch.int32),
                              dev(tables, torch.int32), out, requests, tokens // 64 + requests,
                              heads, kv_heads, head_dim, page_size, num_pages, scale,
                              tensor_core_min, status, tensor_memory=tensor_memory)
    if not tensor_core_min or min(new_tokens) < tensor_core_min:
        ops.paged_attention(dev(q, dtype), dev(to_cache_layout(k_cache, dtype), dtype),
                            dev(to_cache_layout(v_cache, dtype), dtype),
                            dev(positions, torch.int32), dev(token_request, torch.int32),
                            dev(slots, torch.int32), dev(tables, torch.int32), out, partial, tokens,
                            heads, kv_heads, head_dim, page_size, num_pages, window or 0, scale,
                            split_keys, max_splits, status, request_start=starts,
                            skip_query_len=tensor_core_min)
    assert int(status.item()) == (0 if lost_page is None else ops.FLAG_BAD_PAGE)
    expected = []
    for r in range(requests):
        k_r, v_r, offset = keys[r], values[r], contexts[r]
        if lost_keys is not None and lost_keys[0] == r:
            # decode token: it sees every key that is left
            assert new_tokens[r] == 1 and lost_keys[2] <= contexts[r]
            keep = np.r_[0:lost_keys[1], lost_keys[2]:totals[r]]
            k_r, v_r, offset = k_r[:, keep], v_r[:, keep], len(keep) - 1
        context = plain.causal_attention(queries[r], k_r, v_r, query_offset=offset,
                                         window=window or None)
        expected.append(context.transpose(1, 0, 2).reshape(new_tokens[r], heads * head_dim))
    return host(out), np.concatenate(expected), values, positions, token_request


ATTENTION_SHAPES = [
    # heads, kv_heads, head_dim, page_size
    (4, 4, 16, 8), (5, 5, 24, 16), (6, 2, 64, 16), (5, 1, 100, 8), (8, 8, 128, 16), (2, 1, 256, 32),
    (3, 3, 80, 4),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,page_size", ATTENTION_SHAPES)
def test_paged_attention_mixed_batch(dtype, heads, kv_heads, head_dim, page_size):
    rng = np.random.default_rng(7)
    # a prompt from scratch, a continued portion, two single decode tokens (one exactly on a
    # page edge), long enough for several key splits
    contexts = [0, 37, 4 * page_size - 1, 150]
    new_tokens = [45, 19, 1, 1]
    out, expected, *_ = attention_case(rng, dtype, heads, kv_heads, head_dim, page_size, contexts,
                                       new_tokens, window=None, split_keys=64)
    tol = dict(atol=3e-6, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=8e-3)
    assert_close(out, expected, "attention", **tol)


@pytest.mark.parametrize("head_dim", [128, 112, 48, 256])
def test_streaming_attention_row_shared_by_hundreds_of_warps(head_dim):
    """One decode token over 30,000 keys: each of its rows is cut into a few hundred parts
    (more than one merge batch), and one key far inside takes all the weight."""
    rng = np.random.default_rng(21)
    key_position = 12345
    out, expected, values, *_ = attention_case(rng, torch.bfloat16, 2, 2, head_dim, 16, [29999], [1],
                                               window=None, split_keys=64,
                                               dominant={0: key_position})
    assert_close(out, expected, "attention", atol=2e-2, rtol=8e-3)
    wanted = values[0][:, key_position].reshape(1, -1)
    assert_close(out, wanted, "dominant key's value", atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("heads,kv_heads,head_dim,page_size", [
    (3, 3, 64, 8), (4, 2, 128, 32), (2, 2, 16, 8), (3, 1, 48, 16), (2, 2, 80, 32), (4, 2, 96, 8),
    (2, 1, 112, 16), (2, 2, 160, 16), (1, 1, 192, 32), (2, 1, 224, 8), (1, 1, 256, 32)])
def test_streaming_attention_many_requests_of_mixed_length(heads, kv_heads, head_dim, page_size):
    """Seventy requests (more than one group of 32 tokens) with contexts from 0 to 700 keys,
    most decoding one token, some bringing two or three: runs of chunks cross rows, tokens
    and requests everywhere."""
    rng = np.random.default_rng(22)
    contexts = [int(c) for c in rng.integers(0, 700, size=70)]
    contexts[0], contexts[5], contexts[40] = 0, 31, 32
    new_tokens = [1] * 70
    new_tokens[3], new_tokens[33], new_tokens[69] = 2, 3, 2
    out, expected, *_ = attention_case(rng, torch.bfloat16, heads, kv_heads, head_dim, page_size,
                                       contexts, new_tokens, window=None, split_keys=64)
    assert_close(out, expected, "attention", atol=2e-2, rtol=8e-3)


@pytest.mark.parametrize("dtype,window", [(torch.float32, None), (torch.bfloat16, 300)])
def test_attention_with_fewer_splits_than_the_context_needs(dtype, window):
    """``split_keys * max_splits`` smaller than a row's keys: the last split walks on to the end
    of the context, so the result is the same and only less parallel."""
    rng = np.random.default_rng(24)
    out, expected, *_ = attention_case(rng, dtype, 3, 3, 32, 16, [500, 40, 257], [1, 2, 1],
                                       window=window, split_keys=64, max_splits=3)
    tol = dict(atol=3e-6, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=8e-3)
    assert_close(out, expected, "attention", **tol)


@pytest.mark.parametrize("dtype,head_dim", [(torch.bfloat16, 128), (torch.bfloat16, 32),
                                            (torch.float32, 64)])
def test_attention_flags_a_page_outside_the_pool_and_leaves_its_keys_out(dtype, head_dim):
    rng = np.random.default_rng(23)
    out, expected, *_ = attention_case(rng, dtype, 4, 2, head_dim, 16, [10, 200, 70], [1, 1, 1],
                                       window=None, split_keys=64, lost_page=(1, 5))
    assert np.isfinite(out).all()
    tol = dict(atol=3e-6, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=8e-3)
    assert_close(out, expected, "attention without the lost page", **tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 7, 16, 33])
def test_paged_attention_window_edges(dtype, window):
    rng = np.random.default_rng(8)
    out, expected, *_ = attention_case(rng, dtype, 4, 2, 32, 8, [0, 50, 15], [40, 3, 1],
                                       window=window, split_keys=16)
    tol = dict(atol=3e-6, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=8e-3)
    assert_close(out, expected, f"window {window}", **tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key_position", [0, 15, 16, 255, 256, 299])
def test_one_far_key_stands_out(dtype, key_position):
    """One key among 300 is scaled so that it takes all the weight: the output must be that
    key's value, wherever it lies (first key, page edges, split edges, last key)."""
    rng = np.random.default_rng(9)
    out, expected, values, *_ = attention_case(rng, dtype, 4, 4, 32, 16, [299], [1], window=None,
                                               split_keys=64, dominant={0: key_position})
    tol = dict(atol=3e-6, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=8e-3)
    assert_close(out, expected, "attention", **tol)
    wanted = values[0][:, key_position].reshape(1, -1)
    assert_close(out, wanted, "dominant key's value", atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("tensor_memory", [False, True])
@pytest.mark.parametrize("heads,kv_heads,head_dim,page_size", [
    (4, 4, 128, 16), (6, 2, 64, 8), (3, 1, 128, 32), (2, 2, 64, 64), (2, 1, 64, 16),
    (3, 3, 16, 8), (2, 1, 32, 64), (5, 1, 48, 16), (2, 2, 80, 32), (3, 1, 96, 16), (2, 2, 112, 16),
    (2, 1, 160, 16), (1, 1, 192, 8), (2, 2, 224, 32), (2, 1, 256, 32)])
def test_tensor_core_attention_for_prompt_portions(heads, kv_heads, head_dim, page_size,
                                                   tensor_memory):
    if tensor_memory and not ops.prefill_attention_tc_supports(head_dim, page_size):
        pytest.skip("the tcgen05 kernel takes heads of 64 to 128 in steps of 16 and pages of at least 16 keys")
    rng = np.random.default_rng(12)
    # whole prompts (one longer than two tiles, one a single row short of a tile), continued
    # portions that start inside a page and inside a key tile, and two decode tokens that the
    # CUDA-core kernel must fill in beside them
    contexts = [0, 37, 0, 129, 4 * page_size - 1, 70]
    new_tokens = [150, 19, 63, 64, 1, 1]
    out, expected, *_ = attention_case(rng, torch.bfloat16, heads, kv_heads, head_dim, page_size,
                                       contexts, new_tokens, window=None, split_keys=64,
                                       tensor_core_min=16, tensor_memory=tensor_memory)
    assert_close(out, expected, "tensor-core attention", atol=2e-2, rtol=8e-3)


@pytest.mark.parametrize("heads,kv_heads,head_dim,page_size", [(4, 4, 128, 16), (6, 2, 64, 8)])
def test_decode_tokens_between_long_prompt_portions(heads, kv_heads, head_dim, page_size):
    """A serving step: decode tokens and short prompt tails before, between and after prompt
    portions of hundreds of tokens (1,400 tokens in all, 45 rounds of the decode kernel's
    search for its own); the last decode token's far key is scaled to win."""
    rng = np.random.default_rng(17)
    contexts = [130, 0, 999, 512, 40, 77, 64, 301]
    new_tokens = [1, 600, 1, 512, 3, 1, 280, 1]
    far = {7: 123}
    out, expected, values, *_ = attention_case(rng, torch.bfloat16, heads, kv_heads, head_dim,
                                               page_size, contexts, new_tokens, window=None,
                                               split_keys=64, tensor_core_min=16, dominant=far)
    assert_close(out, expected, "attention", atol=2e-2, rtol=8e-3)
    if heads == kv_heads:       # (the key is aimed at one query head of each key head)
        assert_close(out[-1:], values[7][:, far[7]].reshape(1, -1), "far key's value",
                     atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("tensor_memory", [False, True])
def test_prompt_portions_behind_dozens_of_decode_requests(tensor_memory):
    """Forty decode requests come first in the step, as running requests do, and three prompt
    portions behind them: a CTA of the prompt kernels finds its tile among requests 40 to 42,
    beyond the first 32 it looks at."""
    rng = np.random.default_rng(19)
    contexts = [int(c) for c in rng.integers(1, 200, size=40)] + [0, 130, 64]
    new_tokens = [1] * 40 + [300, 100, 70]
    out, expected, *_ = attention_case(rng, torch.bfloat16, 2, 2, 128, 16, contexts, new_tokens,
                                       window=None, split_keys=64, tensor_core_min=64,
                                       tensor_memory=tensor_memory)
    assert_close(out, expected, "attention", atol=2e-2, rtol=8e-3)


@pytest.mark.parametrize("tensor_memory", [False, True])
@pytest.mark.parametrize("key_position", [0, 63, 64, 200, 299])
def test_tensor_core_attention_sees_one_far_key(key_position, tensor_memory):
    rng = np.random.default_rng(13)
    out, expected, values, *_ = attention_case(rng, torch.bfloat16, 4, 4, 128, 16, [270], [30],
                                               window=None, split_keys=64,
                                               dominant={0: key_position}, tensor_core_min=16,
                                               tensor_memory=tensor_memory)
    assert_close(out, expected, "attention", atol=2e-2, rtol=8e-3)
    wanted = values[0][:, key_position].reshape(1, -1)
    assert_close(out[-1:], wanted, "dominant key's value", atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("context", [1024, 2048, 4096])
def test_decode_attention_at_long_contexts(context):
    """Decode tokens over contexts of thousands of keys (the contexts the benchmark and the
    configuration allow), one far key scaled to win, in both precisions: the streaming kernel
    in bfloat16, the CUDA-core kernel with dozens of key splits in float32."""
    for dtype, heads, head_dim in ((torch.bfloat16, 3, 128), (torch.float32, 2, 64)):
        rng = np.random.default_rng(context)
        contexts = [context - 1, context // 2 + 3, 17]
        far = {0: context // 3 + 1}
        out, expected, values, *_ = attention_case(rng, dtype, heads, heads, head_dim, 16, contexts,
                                                   [1, 1, 1], window=None, split_keys=128,
                                                   dominant=far)
        tol = dict(atol=3e-6, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=8e-3)
        assert_close(out, expected, f"attention {dtype}", **tol)
        assert_close(out[:1], values[0][:, far[0]].reshape(1, -1), "far key's value",
                     atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("tensor_memory", [False, True])
@pytest.mark.parametrize("context,new", [(0, 1024), (1024, 1024), (3000, 1096)])
def test_prompt_attention_at_long_contexts(context, new, tensor_memory):
    """Prompt portions whose last rows see 1,024, 2,048 and 4,096 keys, on the ``mma.sync``
    kernel and on the tcgen05 kernel; the last query's far key is scaled to win."""
    rng = np.random.default_rng(context + new)
    heads, head_dim = 2, 128
    far = {0: 777 if context else 5}
    out, expected, values, *_ = attention_case(rng, torch.bfloat16, heads, heads, head_dim, 16,
                                               [context, 40], [new, 70], window=None,
                                               split_keys=64, dominant=far, tensor_core_min=16,
                                               tensor_memory=tensor_memory)
    assert_close(out, expected, "prompt attention", atol=2e-2, rtol=8e-3)
    assert_close(out[new - 1:new], values[0][:, far[0]].reshape(1, -1), "far key's value",
                 atol=2e-2, rtol=1e-2)


def test_tensor_core_attention_refuses_what_it_cannot_tile():
    assert ops.prefill_attention_supports(128, 16) and ops.prefill_attention_supports(64, 64)
    assert ops.prefill_attention_supports(80, 16) and ops.prefill_attention_supports(256, 8)
    # pages of 4 or 24 keys do not tile its 64-key steps, and heads of 72 or 144 are not built:
    # the mixer then takes the CUDA-core kernel, and a direct call is an error, not a wrong
    # result
    for head_dim, page_size in ((64, 4), (128, 24), (72, 16), (144, 16), (8, 16), (288, 16)):
        assert not ops.prefill_attention_supports(head_dim, page_size)
    q = torch.zeros((16, 2 * 64), dtype=torch.bfloat16, device=DEVICE)
    cache = torch.zeros((8, 2, 4, 64), dtype=torch.bfloat16, device=DEVICE)
    zeros = torch.zeros(8, dtype=torch.int32, device=DEVICE)
    with pytest.raises(ops.KernelError, match="pages of 4"):
        ops.prefill_attention(q, cache, cache, zeros, zeros, zeros, zeros.view(1, 8), q.clone(),
                              1, 16, 2, 2, 64, 4, 8, 0.125, 16, status_word())


def test_attention_refuses_odd_head_sizes():
    with pytest.raises(ops.KernelError, match="head_dim"):
        q = torch.zeros((1, 2 * 130), dtype=torch.bfloat16, device=DEVICE)
        cache = torch.zeros((2, 2, 8, 130), dtype=torch.bfloat16, device=DEVICE)
        zeros = torch.zeros(4, dtype=torch.int32, device=DEVICE)
        ops.paged_attention(q, cache, cache, zeros, zeros, zeros, zeros.view(1, 4), q.clone(), None,
                            1, 2, 2, 130, 8, 2, 0, 1.0, 64, 1, status_word())


# -------------------------------------------------------------------- sampling

def test_greedy_takes_the_lowest_id_among_maxima_and_flags_nonfinite_rows():
    rng = np.random.default_rng(10)
    vocab = 1003
    logits = rng.normal(size=(4, vocab)).astype(np.float32)
    logits[0, [700, 30, 999]] = 9.0
    logits[1, vocab - 1] = 50.0
    logits[2, 5] = np.nan
    logits[3, 0] = 11.0
    tokens = torch.zeros(4, dtype=torch.int32, device=DEVICE)
    status = status_word()
    ops.argmax(dev(logits), tokens, status)
    assert tokens.cpu().tolist() == [30, vocab - 1, -1, 0]
    assert int(status.item()) & ops.FLAG_NONFINITE


def test_temperature_sampling_follows_the_inverse_cumulative_distribution():
    rng = np.random.default_rng(11)
    vocab = 777
    rows = 64
    logits = (rng.normal(size=(rows, vocab)) * 2.0).astype(np.float32)
    temperature = np.full(rows, 0.8, dtype=np.float32)
    temperature[0] = 0.0                       # greedy row
    uniform = rng.random(rows).astype(np.float32)
    uniform[1], uniform[2] = 0.0, np.float32(0.999)
    tokens = torch.zeros(rows, dtype=torch.int32, device=DEVICE)
    ops.sample(dev(logits), dev(temperature), dev(uniform), tokens, status_word())
    got = tokens.cpu().numpy()
    assert got[0] == int(np.argmax(logits[0]))
    for row in range(1, rows):
        scaled = (logits[row].astype(np.float64) - logits[row].max()) / temperature[row]
        weights = np.exp(scaled)
        cumulative = np.cumsum(weights)
        target = float(uniform[row]) * cumulative[-1]
        want = int(np.searchsorted(cumulative, target, side="right"))
        want = min(want, vocab - 1)
        if got[row] != want:
            # float32 sums may put a target that lies within rounding of a boundary on the
            # other side of it: accept the neighbour only then
            boundary = cumulative[min(got[row], want)]
            assert abs(got[row] - want) == 1 and abs(target - boundary) < 1e-4 * cumulative[-1], \
                f"row {row}: sampled {got[row]}, expected {want}"
