"""Greedy and temperature sampling of the step's wanted logits, on the device.

Greedy is the reference's rule: lowest id among the maxima, non-finite logits fail the
request (src/model/cpu_generation.cpp:82-97).  The reference samples with nothing else
(docs/MODEL_SUPPORT.md:669-671); temperature sampling is this engine's own:
``p = softmax(logits / T)`` in float32 and the inverse cumulative distribution at a
uniform number drawn from the request's own counter-based stream, keyed by the
request's seed and the index of the token being generated, so a draw never depends
on what else is in the batch or on how the work was cut into steps.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from ..ops import library as ops

_MASK = (1 << 64) - 1


def _splitmix64(value: int) -> int:
    value = (value + 0x9E3779B97F4A7C15) & _MASK
    value = ((value ^ (value >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    value = ((value ^ (value >> 27)) * 0x94D049BB133111EB) & _MASK
    return value ^ (value >> 31)


def uniform_for(seed: int, token_index: int) -> float:
    """The uniform number in [0, 1) for the ``token_index``-th generated token of a request
    with ``seed``: 24 bits of a splitmix64 hash, exact in float32."""
    mixed = _splitmix64((_splitmix64(seed & _MASK) ^ (token_index & _MASK)) & _MASK)
    return (mixed >> 40) / float(1 << 24)


class Sampler:
    def __init__(self, device: torch.device, max_rows: int) -> None:
        self.device = device
        self.max_rows = max_rows
        pin = device.type == "cuda"
        self._host_params = torch.zeros((2, max_rows), dtype=torch.float32, pin_memory=pin)
        self._device_params = torch.zeros((2, max_rows), dtype=torch.float32, device=device)
        self.tokens = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self._host_tokens = torch.zeros(max_rows, dtype=torch.int32, pin_memory=pin)
        self._params_uploaded = torch.cuda.Event() if pin else None
        # results of steps in flight: [tokens..., status word] per slot, with the event that
        # says when the slot has arrived
        self._results = [torch.zeros(max_rows + 1, dtype=torch.int32, pin_memory=pin)
                         for _ in range(2)]
        self._arrived = [torch.cuda.Event() if pin else None for _ in range(2)]

    def prepare(self, temperatures: Sequence[float], uniforms: Sequence[float]) -> bool:
        """Upload the rows' temperatures and uniform numbers; return True when every row is
        greedy (then nothing is uploaded and the arg-max kernel is enough)."""
        rows = len(temperatures)
        if rows > self.max_rows:
            raise ValueError(f"{rows} rows to sample, at most {self.max_rows}")
        if all(t <= 0.0 for t in temperatures):
            return True
        if self._params_uploaded is not None:
            self._params_uploaded.synchronize()     # the last upload has left the pinned block
        params = self._host_params.numpy()
        params[0, :rows] = np.asarray(temperatures, dtype=np.float32)
        params[1, :rows] = np.asarray(uniforms, dtype=np.float32)
        self._device_params.copy_(self._host_params, non_blocking=True)
        if self._params_uploaded is not None:
            self._params_uploaded.record()
        return False

    def launch(self, logits: torch.Tensor, greedy: bool,
               status: Optional[torch.Tensor]) -> torch.Tensor:
        """Select one token per row of ``logits``; returns the device tensor of ids
        (-1: the row held a non-finite logit)."""
        rows = logits.shape[0]
        out = self.tokens[:rows]
        if greedy:
            ops.argmax(logits, out, status)
        else:
            ops.sample(logits, self._device_params[0, :rows], self._device_params[1, :rows], out,
                       status)
        return out

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float],
               uniforms: Sequence[float], status: Optional[torch.Tensor]) -> torch.Tensor:
        return self.launch(logits, self.prepare(temperatures, uniforms), status)

    def to_host(self, tokens: torch.Tensor) -> List[int]:
        rows = tokens.shape[0]
        self._host_tokens[:rows].copy_(tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._host_tokens.numpy()[:rows].tolist()

    def fetch(self, slot: int, tokens: Optional[torch.Tensor], status: torch.Tensor) -> None:
        """Queue the copy of a step's sampled ids (if it sampled) and of the status word to
        the host, behind the step on the current stream; ``collect(slot)`` waits for it.  Two
        slots, so that a step can be queued before the one before it has been collected."""
        result = self._results[slot]
        rows = 0 if tokens is None else tokens.shape[0]
        if rows:
            result[:rows].copy_(tokens, non_blocking=True)
        result[self.max_rows:].copy_(status, non_blocking=True)
        self._arrived[slot].record()

    def collect(self, slot: int, rows: int):
        """Wait for ``fetch(slot, ...)``; returns ``(sampled ids, status flags)``."""
        self._arrived[slot].synchronize()
        values = self._results[slot].numpy()
        return values[:rows].tolist(), int(values[self.max_rows])
