"""``hx_paged_attention_no_alloc`` through its exported C symbol.

Some users of the kernel library cannot give attention a scratch buffer: a server that has
already split all device memory between weights and cache pages, a latency-critical loop
that must not stall the device in ``cudaMalloc``, or a plain-C caller with no allocator of
its own.  For them the library carries the scratch itself (a fixed array in device memory)
and offers this one entry point, which allocates nothing.

The test calls it with ``ctypes`` exactly as such a caller would, twice in a row with
different batches (the second call finds the first call's leftovers in the array), and
compares each result with the ordinary entry point, which is handed freshly allocated
scratch.  It also checks that a batch too large for the built-in array is refused before
anything is launched.  The file sorts last, so a run that stops at the first failure has
already run every other test.
"""
from __future__ import annotations

import ctypes
import math

import numpy as np
import pytest
import torch

from helix_runtime_b200.ops import library as ops

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"
PARTIAL_WORDS = 1 << 20          # HX_NO_ALLOC_PARTIAL_WORDS
COUNTER_WORDS = 1 << 16          # HX_NO_ALLOC_COUNTER_WORDS


def no_alloc_symbol():
    function = ops.lib().hx_paged_attention_no_alloc
    c_int, c_ptr = ctypes.c_int, ctypes.c_void_p
    function.restype = c_int
    function.argtypes = [c_ptr, c_int, c_ptr, c_ptr, c_int, c_ptr, c_ptr, c_ptr, c_ptr, c_int,
                         c_ptr, c_int, c_ptr, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                         c_int, ctypes.c_float, c_int, c_int, c_ptr, c_ptr]
    return function


def make_batch(seed, contexts, heads, head_dim, page_size):
    """Decode tokens of several requests over a shuffled paged cache (bfloat16)."""
    rng = np.random.default_rng(seed)
    requests = len(contexts)
    pages_per = [-(-(c + 1) // page_size) for c in contexts]
    num_pages = sum(pages_per) + 2
    order = rng.permutation(num_pages)
    tables = np.full((requests, max(pages_per)), -1, dtype=np.int32)
    cursor = 0
    for r in range(requests):
        tables[r, :pages_per[r]] = order[cursor:cursor + pages_per[r]]
        cursor += pages_per[r]

    def tensor(array, dtype):
        return torch.as_tensor(np.asarray(array)).to(device=DEVICE, dtype=dtype).contiguous()

    cache_shape = (num_pages, heads, page_size, head_dim)
    return dict(
        q=tensor(rng.normal(size=(requests, heads * head_dim)), torch.bfloat16),
        keys=tensor(rng.normal(size=cache_shape), torch.bfloat16),
        values=tensor(rng.normal(size=cache_shape), torch.bfloat16),
        positions=tensor(contexts, torch.int32),
        token_request=tensor(np.arange(requests), torch.int32),
        rows=tensor(np.arange(requests), torch.int32),
        tables=tensor(tables, torch.int32),
        tokens=requests, heads=heads, head_dim=head_dim, page_size=page_size,
        num_pages=num_pages, longest=max(contexts) + 1)


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
                        batch["page_size"], batch["num_pages"], 0,
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
        batch["values"].data_ptr(), ops.HX_BF16, batch["positions"].data_ptr(),
        batch["token_request"].data_ptr(), batch["rows"].data_ptr(), batch["tables"].data_ptr(),
        batch["tables"].stride(0), None, 0, out.data_ptr(), out.stride(0),
        tokens or batch["tokens"], batch["heads"], batch["heads"], head_dim or batch["head_dim"],
        batch["page_size"], batch["num_pages"], 0, 1.0 / math.sqrt(batch["head_dim"]), split_keys,
        max_splits, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return code, out.float().cpu().numpy(), int(status.item())


def test_two_calls_in_a_row_match_the_ordinary_entry_point():
    torch.cuda.synchronize()
    # the first call also does the per-device set-up (outside of any stream capture)
    first = make_batch(1, contexts=[300, 17, 129, 255, 64], heads=6, head_dim=128, page_size=16)
    second = make_batch(2, contexts=[40, 700], heads=3, head_dim=64, page_size=8)
    for batch, split_keys in ((first, 64), (second, 32)):
        expected = run_ordinary(batch, split_keys)
        before = torch.cuda.memory_allocated()
        code, got, flags = run_no_alloc(batch, split_keys)
        assert code == 0, ops.lib().hx_last_error().decode()
        assert flags == 0
        assert np.isfinite(got).all()
        # the tolerance the kernel tests use for bfloat16 outputs
        np.testing.assert_allclose(got, expected, atol=2e-2, rtol=8e-3)
        assert torch.cuda.memory_allocated() <= before + got.nbytes   # only the output tensor


def test_a_batch_beyond_the_built_in_array_is_refused_before_any_launch():
    batch = make_batch(3, contexts=[100, 200], heads=4, head_dim=128, page_size=16)
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
