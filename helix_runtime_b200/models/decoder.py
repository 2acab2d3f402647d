"""A decoder assembled from a :class:`ModelSpec`: embedding, scheduled blocks, norm, head.

The model owns the parts and the order in which they run; it owns no cache and no
batch.  ``forward`` runs exactly the tokens of the step's context through every
schedule entry and returns float32 logits at the wanted rows.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Mapping, Optional, Sequence

import torch

from ..cache.manager import CacheManager, KvNeed, StateNeed
from ..config.spec import BlockSpec, ModelSpec
from ..parts.base import (FeedForward, LayerCache, Mixer, Norm, StepContext, build_part)
from ..weights.loader import TensorRequest


# ----------------------------------------------------------------- arrangements
#
# An arrangement wires the parts of a block: ``run(block, ctx, cache, residual, normed)`` reads
# and updates the float32 residual stream ``residual[:n]`` through the block's parts, with
# ``normed`` as scratch for a norm's output (compute dtype, same rows).  Mixers and
# feed-forwards ADD their output into the residual they are handed.

Arrangement = Callable[["Block", StepContext, LayerCache, torch.Tensor, torch.Tensor], None]
_ARRANGEMENTS: Dict[str, Arrangement] = {}


def register_arrangement(name: str, run: Arrangement) -> None:
    """Make ``name`` usable as ``BlockSpec.arrangement``."""
    _ARRANGEMENTS[name] = run


def _pre_norm(block: "Block", ctx: StepContext, cache: LayerCache, residual: torch.Tensor,
              normed: torch.Tensor) -> None:
    # x += mixer(norm(x)); x += ff(norm(x))   (src/model/cpu_llama.cpp:62-98)
    block.mixer_norm.forward(ctx, residual, normed)
    block.mixer.forward(ctx, cache, normed, residual)
    if block.feed_forward is not None:
        block.feed_forward_norm.forward(ctx, residual, normed)
        block.feed_forward.forward(ctx, normed, residual)


register_arrangement("pre_norm", _pre_norm)


class Block:
    """One decoder layer: its parts, and the arrangement that runs them."""

    def __init__(self, spec: BlockSpec, hidden_size: int) -> None:
        run = _ARRANGEMENTS.get(spec.arrangement)
        if run is None:
            raise ValueError(f"unknown block arrangement {spec.arrangement!r}; known: "
                             + ", ".join(sorted(_ARRANGEMENTS)))
        if (spec.feed_forward is None) != (spec.feed_forward_norm is None) \
                and spec.arrangement == "pre_norm":
            raise ValueError("a pre_norm block has a feed-forward with its norm, or neither")
        self.arrangement = spec.arrangement
        self._run = run
        self.mixer_norm: Norm = build_part("norm", spec.mixer_norm, hidden_size)
        self.mixer: Mixer = build_part("mixer", spec.mixer, hidden_size)
        self.feed_forward_norm: Optional[Norm] = None if spec.feed_forward_norm is None else \
            build_part("norm", spec.feed_forward_norm, hidden_size)
        self.feed_forward: Optional[FeedForward] = None if spec.feed_forward is None else \
            build_part("feed_forward", spec.feed_forward, hidden_size)

    def parts(self):
        return tuple(part for part in (self.mixer_norm, self.mixer, self.feed_forward_norm,
                                       self.feed_forward) if part is not None)

    def forward(self, ctx: StepContext, cache: LayerCache, residual: torch.Tensor,
                normed: torch.Tensor) -> None:
        self._run(self, ctx, cache, residual, normed)


class DecoderModel:
    def __init__(self, spec: ModelSpec) -> None:
        spec.validate()
        self.spec = spec
        self.hidden_size = spec.hidden_size
        self.vocab_size = spec.vocab_size
        self.max_positions = spec.max_positions
        self.embedding = build_part("embedding", spec.embedding, spec.hidden_size)
        self.blocks: List[Block] = [Block(block, spec.hidden_size) for block in spec.blocks]
        self.schedule = spec.schedule
        self.final_norm: Norm = build_part("norm", spec.final_norm, spec.hidden_size)
        self.lm_head = build_part("lm_head", spec.lm_head, spec.hidden_size)
        self.dtype: Optional[torch.dtype] = None
        self.device: Optional[torch.device] = None

    # ------------------------------------------------------------------ weights

    def all_parts(self):
        yield self.embedding
        for block in self.blocks:
            yield from block.parts()
        yield self.final_norm
        yield self.lm_head

    @property
    def graph_safe(self) -> bool:
        """Whether every part may be recorded into a CUDA graph (see ``Part.graph_safe``)."""
        return all(part.graph_safe for part in self.all_parts())

    def tensor_requests(self) -> List[TensorRequest]:
        requests: List[TensorRequest] = []
        seen = set()
        for part in self.all_parts():
            for request in part.tensor_requests():
                if request.name not in seen:
                    seen.add(request.name)
                    requests.append(request)
        return requests

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype,
             device: torch.device) -> None:
        for part in self.all_parts():
            part.bind(tensors, dtype, device)
        self.dtype = dtype
        self.device = device

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights one step reads: every matrix and norm of every scheduled layer once,
        plus the head (the embedding is gathered, not streamed)."""
        total = self.final_norm.weight_bytes() + self.lm_head.weight_bytes()
        for entry in self.schedule:
            total += sum(part.weight_bytes() for part in self.blocks[entry.block].parts())
        return total

    # -------------------------------------------------------------------- cache

    def cache_needs(self):
        """``(kv_needs, state_needs)`` keyed by the schedule entries that own a cache."""
        kv: Dict[int, KvNeed] = {}
        state: Dict[int, StateNeed] = {}
        for index, entry in enumerate(self.schedule):
            if entry.cache_from is not None:
                continue
            mixer = self.blocks[entry.block].mixer
            need = mixer.kv_need()
            if need is not None:
                kv[index] = need
            state_need = mixer.state_need()
            if state_need is not None:
                state[index] = state_need
        for index, entry in enumerate(self.schedule):
            if entry.cache_from is None:
                continue
            own = self.blocks[entry.block].mixer.kv_need()
            other = self.blocks[self.schedule[entry.cache_from].block].mixer.kv_need()
            if own != other:
                raise ValueError(f"schedule entry {index} reads the cache of entry "
                                 f"{entry.cache_from}, whose geometry differs")
        return kv, state

    def layer_cache(self, cache: CacheManager, index: int) -> LayerCache:
        entry = self.schedule[index]
        owner = index if entry.cache_from is None else entry.cache_from
        view = LayerCache(entry=owner, owns=entry.cache_from is None)
        if cache.owns_pages(owner):
            group = cache.group_of(owner)
            view.keys, view.values = cache.layer_storage(owner)
            view.block_tables = group.device_tables
            view.page_size = group.page_size
            view.num_pages = group.pool.num_pages
            view.window = group.need.window
        if owner in cache.states:
            view.state = cache.state(owner)
        return view

    # ------------------------------------------------------------------ forward

    def forward(self, ctx: StepContext, cache: CacheManager, want_rows: Optional[torch.Tensor],
                n_want: int) -> Optional[torch.Tensor]:
        """Run the step's tokens; return logits ``[n_want, vocab]`` float32 for the flattened
        token indices in ``want_rows`` (device int32), or None when nothing is wanted."""
        h = self.hidden_size
        residual = ctx.workspace.get("model.residual", (ctx.capacity, h), torch.float32)
        normed = ctx.workspace.get("model.normed", (ctx.capacity, h), ctx.dtype)
        self.embedding.forward(ctx, residual)
        for index, entry in enumerate(self.schedule):
            self.blocks[entry.block].forward(ctx, self.layer_cache(cache, index), residual, normed)
        if n_want == 0:
            return None
        wanted = ctx.workspace.get("model.wanted", (ctx.capacity, h), ctx.dtype)
        logits = ctx.workspace.get("model.logits", (ctx.capacity, self.vocab_size), torch.float32)
        self.final_norm.forward(ctx, residual, wanted, rows=want_rows, n_rows=n_want)
        self.lm_head.forward(ctx, wanted, logits, n_want)
        return logits[:n_want]
