"""``hx_paged_attention_no_alloc`` through its exported C symbol.

Some users of the kernel library cannot give attention a scratch buffer: a server that has
already split all device memory between weights and cache pages, a latency-critical loop
that must not stall the device in ``cudaMalloc``, or a plain-C caller with no allocator of
its own.  For them the library carries the scratch itself (a fixed array in device memory)
and offers this one entry point, which allocates nothing.

The tests call it with ``ctypes`` exactly as such a caller would, several times in a row
with different batches (every call finds the leftovers of the one before in the array),
and compare each result with the ordinary entry point, which is handed freshly allocated
scratch, and with the plain float64 attention of ``plain_llama`` (the two entry points run
the same kernels, so only the plain one can show a wrong result that both share).  The
cases cover both kinds of scratch use: the streaming kernel's two parts per warp
(bfloat16, up to 256-wide heads) and the CUDA-core kernel's part per key split with its
arrival counters (float32, and bfloat16 with a window).  A batch too large for the built-in
array is refused before anything is launched.  The file sorts last, so a run that stops at
the first failure has already run every other test.
"""
from __future__ import annotations

import ctypes
import math

import numpy as np
import pytest
import torch

import plain_llama as plain
from helix_runtime_b200.ops import library as ops

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"
PARTIAL_WORDS = 17 << 16         # HX_NO_ALLOC_PARTIAL_WORDS
COUNTER_WORDS = 1 << 16          # HX_NO_ALLOC_COUNTER_WORDS


def no_alloc_symbol():
    function = ops.lib().hx_paged_attention_no_alloc
    c_int, c_ptr = ctypes.c_int, ctypes.c_void_p
    function.restype = c_int
    function.argtypes = [c_ptr, c_int, c_ptr, c_ptr, c_int, c_ptr, c_ptr, c_ptr, c_ptr, c_int,
                         c_ptr, c_int, c_ptr, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                         c_int, ctypes.c_float, c_int, c_int, c_ptr, c_ptr]
    return function


def cache_layout(rows, chunk):
    """[page, head, slot, dim] -> the cache's [page, head, dim / chunk, slot, chunk]."""
    pages, heads, slots, dim = rows.shape
    return rows.reshape(pages, heads, slots, dim // chunk, chunk).transpose(0, 1, 3, 2, 4) \
        .reshape(rows.shape)


def make_batch(seed, contexts, heads, head_dim, page_size, dtype=torch.bfloat16, window=0):
    """Decode tokens of several requests over a shuffled paged cache.  ``expected`` is the
    plain float64 attention over the values the tensors really hold."""
    rng = np.random.default_rng(seed)
    requests = len(contexts)
    pages_per = [-(-(c + 1) // page_size) for c in contexts]
    num_pages = sum(pages_per) + 2
    order = rng.permutation(num_pages)
    tables = np.full((requests, max(pages_per)), -1, dtype=np.int32)

    def tensor(array, kind):
        return torch.as_tensor(np.asarray(array)).to(device=DEVICE, dtype=kind).contiguous()

    def held(array):
        return tensor(array, dtype).float().cpu().numpy()

    queries = held(rng.normal(size=(requests, heads, head_dim)))
    k_rows = np.full((num_pages, heads, page_size, head_dim), np.nan, dtype=np.float32)
    v_rows = np.full_like(k_rows, np.nan)
    expected = []
    cursor = 0
    for r, context in enumerate(contexts):
        total = context + 1
        keys = held(rng.normal(size=(heads, total, head_dim)))
        values = held(rng.normal(size=(heads, total, head_dim)))
        for p in range(pages_per[r]):
            page = order[cursor]
            cursor += 1
            tables[r, p] = page
            lo, hi = p * page_size, min((p + 1) * page_size, total)
            k_rows[page, :, :hi - lo] = keys[:, lo:hi]
            v_rows[page, :, :hi - lo] = values[:, lo:hi]
        context_rows = plain.causal_attention(queries[r][:, None, :], keys, values,
                                              query_offset=context, window=window or None)
        expected.append(context_rows.reshape(1, heads * head_dim))
    chunk = ops.lib().hx_cache_chunk_elements(ops.HX_BF16 if dtype == torch.bfloat16
                                              else ops.HX_F32, head_dim)
    return dict(
        q=tensor(queries.reshape(requests, heads * head_dim), dtype),
        keys=tensor(cache_layout(k_rows, chunk), dtype),
        values=tensor(cache_layout(v_rows, chunk), dtype),
        positions=tensor(contexts, torch.int32),
        token_request=tensor(np.arange(requests), torch.int32),
        rows=tensor(np.arange(requests), torch.int32),
        tables=tensor(tables, torch.int32),
        tokens=requests, heads=heads, head_dim=head_dim, page_size=page_size,
        num_pages=num_pages, window=window, dtype=dtype,
        code=ops.HX_BF16 if dtype == torch.bfloat16 else ops.HX_F32,
        longest=min(max(contexts) + 1, window) if window else max(contexts) + 1,
        expected=np.concatenate(expected))


def run_ordinary(batch, split_keys):
    max_splits = -(-batch["longest"] // split_keys)
    out = torch.full_like(batch["q"], float("nan"))
    partial = torch.empty(ops.attention_scratch_floats(batch["tokens"], batch["heads"],
                                                       batch["head_dim"], max_splits),
                          dtype=torch.float32, device=DEVICE)
    status = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    ops.paged_attention(batch["q"], batch["keys"], batch["values"], batch["positions"],
                        batch["token_request"], batch["rows"], batch["tables"], out, partial,
                        batch["tokens"], batch["heads"], batch["heads"], batch["head_dim"],
                        batch["page_size"], batch["num_pages"], batch["window"],
                        1.0 / math.sqrt(batch["head_dim"]), split_keys, max_splits, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return out.float().cpu().numpy()


def run_no_alloc(batch, split_keys, tokens=None, max_splits=None, head_dim=None):
    max_splits = max_splits or -(-batch["longest"] // split_keys)
    out = torch.full_like(batch["q"], float("nan"))
    status = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    code = no_alloc_symbol()(
        batch["q"].data_ptr(), batch["q"].stride(0), batch["keys"].data_ptr(),
        batch["values"].data_ptr(), batch["code"], batch["positions"].data_ptr(),
        batch["token_request"].data_ptr(), batch["rows"].data_ptr(), batch["tables"].data_ptr(),
        batch["tables"].stride(0), None, 0, out.data_ptr(), out.stride(0),
        tokens or batch["tokens"], batch["heads"], batch["heads"], head_dim or batch["head_dim"],
        batch["page_size"], batch["num_pages"], batch["window"],
        1.0 / math.sqrt(batch["head_dim"]), split_keys, max_splits, status.data_ptr(),
        torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return code, out.float().cpu().numpy(), int(status.item())


def check_calls_in_a_row(cases):
    """Every case through the no-alloc entry point, one after the other, each against the
    ordinary entry point and against the plain attention."""
    torch.cuda.synchronize()
    for batch, split_keys in cases:
        ordinary = run_ordinary(batch, split_keys)
        before = torch.cuda.memory_allocated()
        code, got, flags = run_no_alloc(batch, split_keys)
        assert code == 0, ops.lib().hx_last_error().decode()
        assert flags == 0
        assert np.isfinite(got).all()
        assert torch.cuda.memory_allocated() <= before + got.nbytes   # only the output tensor
        # the tolerances the kernel tests use for attention outputs
        tol = dict(atol=3e-6, rtol=1e-5) if batch["dtype"] == torch.float32 \
            else dict(atol=2e-2, rtol=8e-3)
        np.testing.assert_allclose(got, ordinary, **tol)
        np.testing.assert_allclose(got, batch["expected"], **tol)


def test_two_calls_in_a_row_match_the_ordinary_entry_point():
    # the first call also does the per-device set-up (outside of any stream capture)
    first = make_batch(1, contexts=[300, 17, 129, 255, 64], heads=6, head_dim=128, page_size=16)
    second = make_batch(2, contexts=[40, 700], heads=3, head_dim=64, page_size=8)
    check_calls_in_a_row(((first, 64), (second, 32)))


def test_key_splits_with_arrival_counters_use_the_built_in_array():
    """float32 and a windowed bfloat16 batch go to the CUDA-core kernel, whose splits write a
    part each and count arrivals in the built-in array; a second call of each follows a call
    that left other parts and (cleared) counters behind."""
    single = make_batch(4, contexts=[500, 33, 260], heads=3, head_dim=48, page_size=16,
                        dtype=torch.float32)
    windowed = make_batch(5, contexts=[400, 90, 257], heads=4, head_dim=64, page_size=16,
                          window=200)
    again = make_batch(6, contexts=[131, 402], heads=5, head_dim=24, page_size=8,
                       dtype=torch.float32)
    check_calls_in_a_row(((single, 64), (windowed, 32), (again, 32), (windowed, 64)))


def test_heads_of_256_fit_the_built_in_array():
    wide = make_batch(7, contexts=[300, 70, 1000], heads=2, head_dim=256, page_size=16)
    narrow = make_batch(8, contexts=[45, 610], heads=2, head_dim=160, page_size=32)
    check_calls_in_a_row(((wide, 64), (narrow, 64), (wide, 128)))


def test_a_batch_beyond_the_built_in_array_is_refused_before_any_launch():
    # float32 is served by the CUDA-core kernel, whose scratch grows with tokens and splits
    batch = make_batch(3, contexts=[100, 200], heads=4, head_dim=128, page_size=16,
                       dtype=torch.float32)
    # pretend to many more tokens and splits than the scratch can serve: nothing may run, so the
    # pointers are never followed
    tokens, max_splits = 4096, 64
    assert tokens * 4 * max_splits * 130 > PARTIAL_WORDS
    code, out, flags = run_no_alloc(batch, 64, tokens=tokens, max_splits=max_splits)
    assert code != 0 and flags == 0
    message = ops.lib().hx_last_error().decode()
    assert "words of scratch" in message and str(PARTIAL_WORDS) in message
    assert np.isnan(out).all()                  # the output was not touched
    # tiny heads: the partial sums fit, the counters (one per token and head) do not
    tokens = COUNTER_WORDS // 4 + 1
    assert tokens * 4 * 2 * (2 + 2) <= PARTIAL_WORDS
    code, out, flags = run_no_alloc(batch, 64, tokens=tokens, max_splits=2, head_dim=2)
    assert code != 0 and "arrival counters" in ops.lib().hx_last_error().decode()
    assert np.isnan(out).all()
