"""A small in-process driver of the engine's own model, cache and step function for tests."""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from helix_runtime_b200.cache.manager import CacheManager
from helix_runtime_b200.engine.engine import load_model
from helix_runtime_b200.engine.step import StepEntry, StepFunction

# Logits of the tiny models have a spread of about 0.2.
# float32: the engine accumulates in float32 where the plain implementation uses double; the
# reference allows 5e-5 between its CPU model and its oracle and 2e-4 between CUDA and CPU
# (tests/llama_model_test.cpp, tests/cuda_llama_model_test.cpp:20-21).
F32_TOL = dict(atol=2e-5, rtol=1e-4)
# bfloat16: the plain implementation rounds activations to bfloat16 at the places where the
# engine stores them, so what is left is float32-vs-double summation and activations that fall
# on the other side of a rounding boundary (one part in 256 of that activation), which the
# sharpened attention and the final norm carry into the logits.  For scale: rounding to
# bfloat16 itself moves the logits of these models by up to 2e-2.
BF16_TOL = dict(atol=5e-3, rtol=5e-3)
# The wider model C has larger logits (spread 0.32) and more terms per sum, and rounding to
# bfloat16 itself moves its logits more: measured with the plain implementation (float32
# against rounded, 150 and 300 tokens) the largest change is 3.6e-3 for A, 6.6e-3 for B and
# 1.14e-2 for C.  Its absolute tolerance is 0.8 of that change, as for B.
BF16_ATOL_BY_MODEL = {"C": 9e-3}


def tolerance(dtype: str, name: str = "") -> dict:
    if dtype == "float32":
        return F32_TOL
    return dict(BF16_TOL, atol=BF16_ATOL_BY_MODEL.get(name, BF16_TOL["atol"]))


class Harness:
    def __init__(self, folder: str, dtype: str, page_size: int, num_pages: int,
                 max_requests: int = 4, max_tokens: int = 512, split_keys: int = 256,
                 poison: bool = True) -> None:
        self.model = load_model(folder, dtype, "cuda:0")
        kv, state = self.model.cache_needs()
        self.cache = CacheManager(kv, state, page_size, num_pages, max_requests,
                                  self.model.max_positions, self.model.dtype,
                                  torch.device("cuda:0"), poison=poison)
        self.step = StepFunction(self.model, self.cache, max_tokens, max_requests,
                                 attention_split_keys=split_keys)

    def run(self, entries: Sequence[Tuple[Hashable, Sequence[int], Sequence[int]]]) -> Optional[np.ndarray]:
        batch = []
        for request, tokens, want in entries:
            if not self.cache.has(request):
                self.cache.admit(request)
            batch.append(StepEntry(request, list(tokens), list(want)))
        logits = self.step.run(batch)
        return None if logits is None else logits.float().cpu().numpy().copy()

    def end(self, request: Hashable) -> None:
        self.cache.release(request)

    def whole(self, request: Hashable, tokens: Sequence[int]) -> np.ndarray:
        """Every position's logits from one step; the request is released afterwards."""
        out = self.run([(request, tokens, range(len(tokens)))])
        self.end(request)
        return out


def assert_close(actual: np.ndarray, expected: np.ndarray, what: str, atol: float, rtol: float) -> None:
    assert actual.shape == expected.shape, f"{what}: shape {actual.shape} vs {expected.shape}"
    assert np.isfinite(actual).all(), f"{what}: non-finite values"
    error = np.abs(actual.astype(np.float64) - expected.astype(np.float64))
    bound = atol + rtol * np.abs(expected.astype(np.float64))
    if (error > bound).any():
        worst = np.unravel_index(np.argmax(error - bound), error.shape)
        rows = sorted(set(np.argwhere(error > bound)[:, 0].tolist()))
        raise AssertionError(
            f"{what}: {int((error > bound).sum())} of {error.size} values differ; worst at "
            f"{tuple(int(i) for i in worst)}: {actual[worst]!r} vs {expected[worst]!r} "
            f"(error {error[worst]:.3e}, allowed {bound[worst]:.3e}); first bad row {rows[0]}, "
            f"bad rows {rows[:12]}")
