"""Interfaces of the parts a decoder layer is made of, and the registry that builds them.

A part is built from its :class:`~helix_runtime_b200.config.PartSpec` alone: every
size and constant is a parameter, the checkpoint tensor names it binds are
parameters too, and no part knows which model it is in.  The life of a part:

1. ``Part(spec, hidden_size)`` — construction from data;
2. ``tensor_requests()`` — which checkpoint tensors it binds, with shapes and roles;
3. ``bind(tensors, dtype, device)`` — take the loaded tensors, do load-time layout
   work (fusing, permuting), keep device tensors;
4. ``forward(...)`` once per step, launching kernels on the current stream.

Interfaces (all tensors live on the device; ``ctx`` is the step's
:class:`StepContext`):

* Norm:          ``forward(ctx, x_f32[N,H], out[N,H], rows=None)`` writes the compute dtype.
* Mixer:         ``forward(ctx, cache, x[N,H], residual_f32[N,H])`` adds its output into
  ``residual``.  ``kv_need()`` / ``state_need()`` say what it wants of the cache manager;
  ``cache`` is the :class:`LayerCache` of the schedule entry being run.
* FeedForward:   ``forward(ctx, x[N,H], residual_f32[N,H])`` adds its output into ``residual``.
* PositionEncoding: owned by a mixer; ``apply(ctx, cache, qkv, ...)`` encodes queries and
  keys in place and stores keys/values into the cache pages.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, Dict, List, Mapping, Optional, Tuple

import torch

from ..cache.manager import KvNeed, StateNeed
from ..config.spec import PartSpec
from ..weights.loader import TensorRequest


class Workspace:
    """Named scratch tensors that keep their address from step to step.

    A buffer is created at its first use with the capacity the step function was
    built for and handed out again under the same name, so a captured CUDA graph can
    be replayed against the same memory.  A buffer that has to be replaced (another
    shape under the same name, a flat buffer that must grow) is kept alive beside its
    successor: graphs recorded earlier still point at it, and it is as large as they
    need."""

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self._buffers: Dict[str, torch.Tensor] = {}
        self._accumulators: Dict[str, torch.Tensor] = {}
        self._retired: List[torch.Tensor] = []
        self._retired_accumulators: List[torch.Tensor] = []

    def _replace(self, table: Dict[str, torch.Tensor], name: str, buffer: torch.Tensor) -> None:
        old = table.get(name)
        if old is not None:
            (self._retired_accumulators if table is self._accumulators
             else self._retired).append(old)
        table[name] = buffer

    def get(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        buffer = self._buffers.get(name)
        if buffer is None or buffer.dtype != dtype or tuple(buffer.shape) != tuple(shape):
            buffer = torch.empty(shape, dtype=dtype, device=self.device)
            self._replace(self._buffers, name, buffer)
        return buffer

    def accumulator(self, name: str, shape: Tuple[int, ...],
                    dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """A buffer that is all zero whenever nobody is using it: kernels that sum into it
        (split-K products, arrival counters) are followed by code that clears it again."""
        buffer = self._accumulators.get(name)
        if buffer is None or tuple(buffer.shape) != tuple(shape) or buffer.dtype != dtype:
            buffer = torch.zeros(shape, dtype=dtype, device=self.device)
            self._replace(self._accumulators, name, buffer)
        return buffer

    def clear_accumulators(self) -> None:
        """After a step that failed half-way: restore the all-zero state."""
        for buffer in (*self._accumulators.values(), *self._retired_accumulators):
            buffer.zero_()

    def at_least(self, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """A flat buffer of at least ``numel`` elements.  It grows by doubling at least, so
        that the buffers it leaves behind stay a fraction of its size."""
        buffer = self._buffers.get(name)
        if buffer is None or buffer.dtype != dtype or buffer.numel() < numel:
            if buffer is not None and buffer.dtype == dtype:
                numel = max(numel, 2 * buffer.numel())
            buffer = torch.empty((numel,), dtype=dtype, device=self.device)
            self._replace(self._buffers, name, buffer)
        return buffer

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size()
                   for t in (*self._buffers.values(), *self._accumulators.values(),
                             *self._retired, *self._retired_accumulators))


@dataclasses.dataclass
class LayerCache:
    """What one schedule entry sees of the cache manager."""
    entry: int                                  # the schedule entry that owns the storage
    owns: bool                                  # False: reads another entry's cache, writes nothing
    keys: Optional[torch.Tensor] = None         # [page, kv_head, (head_dim/c, slot, c)]: chunked
    values: Optional[torch.Tensor] = None
    block_tables: Optional[torch.Tensor] = None  # [state slot, page index] int32
    page_size: int = 0
    num_pages: int = 0
    window: Optional[int] = None
    state: Optional[torch.Tensor] = None        # [state slot, *shape]


@dataclasses.dataclass
class StepContext:
    """One step's batch as the parts see it.  N tokens of R requests, flattened."""
    dtype: torch.dtype
    device: torch.device
    workspace: Workspace
    capacity: int                       # rows of every workspace activation buffer
    n_tokens: int
    n_requests: int
    token_ids: torch.Tensor             # [capacity] int32
    positions: torch.Tensor             # [capacity] int32 absolute position of each token
    token_request: torch.Tensor         # [capacity] int32 index into the step's requests
    request_slot: torch.Tensor          # [max requests] int32 state slot / block table row
    request_start: torch.Tensor         # [max requests + 1] int32 first token of each request
    request_context: torch.Tensor       # [max requests] int32 tokens cached before this step
    status: torch.Tensor                # [1] int32 device status word
    max_query_len: int                  # host copies, for grid sizing
    min_query_len: int                  # fewest tokens any request brings to this step
    max_context_len: int                # longest (cached + new) length in the batch
    attention_split_keys: int = 256
    ordered_sums: bool = False          # products must sum in a fixed order (no split-K atomics)
    # host-side copies for parts that are not kernels (tests' toy parts)
    host_request_slots: Optional[List[int]] = None
    host_request_starts: Optional[List[int]] = None
    host_request_contexts: Optional[List[int]] = None
    host_query_lengths: Optional[List[int]] = None      # tokens each request brings


class Part:
    # Decode steps are recorded into CUDA graphs and replayed.  A part whose forward reads
    # device values on the host (``.item()``, ``nonzero()``, a loop over requests) cannot be
    # recorded: it says so here, and the engine then runs every step of its model eagerly.
    graph_safe: bool = True

    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        self.spec = spec
        self.hidden_size = hidden_size

    def tensor_requests(self) -> List[TensorRequest]:
        return []

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype,
             device: torch.device) -> None:
        pass

    def weight_bytes(self) -> int:
        """Bytes of weights a step reads from this part (for roofline accounting)."""
        return 0


class Norm(Part):
    def forward(self, ctx: StepContext, x: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    """Owned by a mixer, which calls :meth:`apply` on the projected rows of a step."""

    # How the encoding pairs coordinates, if it pairs them at all ("adjacent", "half_split"):
    # a mixer whose checkpoint rows are laid out for another pairing permutes them at load.
    pairing: Optional[str] = None

    def apply(self, ctx: "StepContext", cache: "LayerCache", qkv: torch.Tensor, heads: int,
              kv_heads: int, accum: Optional[torch.Tensor] = None) -> None:
        """Encode queries and keys of ``qkv[:ctx.n_tokens]`` (rows ``[q heads | k heads |
        v heads]``) in place and store keys and values into the entry's pages when
        ``cache.owns``.  With ``accum`` the projection arrives in that float32 accumulator
        instead of ``qkv`` and the accumulator must be left cleared."""
        raise NotImplementedError

    def project_and_apply(self, ctx: "StepContext", cache: "LayerCache", x: torch.Tensor,
                          weight, qkv: torch.Tensor, heads: int, kv_heads: int) -> bool:
        """Optional: the mixer's projection ``qkv[:n] = x[:n] @ weight.T`` and :meth:`apply`
        as ONE kernel.  Return False (the default) when this encoding has no such kernel for
        this step; the mixer then projects and calls :meth:`apply`.  After a True only the
        query columns of ``qkv`` are defined: keys and values live in the pages."""
        return False


class Mixer(Part):
    def kv_need(self) -> Optional[KvNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, ctx: StepContext, cache: LayerCache, x: torch.Tensor,
                residual: torch.Tensor) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx: StepContext, x: torch.Tensor, residual: torch.Tensor) -> None:
        raise NotImplementedError


# ------------------------------------------------------------------- registry

_REGISTRY: Dict[Tuple[str, str], Callable[[PartSpec, int], Part]] = {}
_FAMILIES = ("norm", "position", "mixer", "feed_forward", "embedding", "lm_head")


def register_part(family: str, kind: str, factory: Callable[[PartSpec, int], Part]) -> None:
    """Make ``kind`` buildable.  ``family`` is one of norm, position, mixer, feed_forward,
    embedding, lm_head; ``factory(spec, hidden_size)`` returns the part."""
    if family not in _FAMILIES:
        raise ValueError(f"unknown part family {family!r}; known: {', '.join(_FAMILIES)}")
    _REGISTRY[(family, kind)] = factory


def build_part(family: str, spec: PartSpec, hidden_size: int) -> Part:
    factory = _REGISTRY.get((family, spec.kind))
    if factory is None:
        known = sorted(kind for fam, kind in _REGISTRY if fam == family)
        raise KeyError(f"no {family} part of kind {spec.kind!r}; known: {', '.join(known)}")
    return factory(spec, hidden_size)


def registered_parts() -> List[Tuple[str, str]]:
    return sorted(_REGISTRY)
