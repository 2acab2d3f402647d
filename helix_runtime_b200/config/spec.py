"""Architecture-neutral description of a decoder: which parts each layer is made of.

An architecture's typed configuration (read from its own ``config.json`` keys) is
translated into a :class:`ModelSpec` by that architecture's ``build_spec``.  The
spec is plain data: every size and constant a part needs is a field of its spec,
the blocks are a list (one :class:`BlockSpec` per distinct layer), and the order
in which layers run is a second list (:class:`ScheduleEntry`), which may name a
block twice or let an entry read the cache written by an earlier entry.

The reference hard-wires this structure into one function
(src/model/cpu_llama.cpp:62-98); here it is data so that a second architecture
only adds a new ``build_spec``.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Mapping, Optional, Tuple


@dataclasses.dataclass(frozen=True)
class PartSpec:
    """A part's kind (the key in the part registry) plus its parameters."""

    kind: str
    params: Mapping[str, Any] = dataclasses.field(default_factory=dict)
    # checkpoint tensor names this part binds, keyed by the part's own role names
    tensors: Mapping[str, str] = dataclasses.field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclasses.dataclass(frozen=True)
class BlockSpec:
    """One decoder layer: a mixer and (usually) a feed-forward, each behind its own norm.

    ``arrangement`` names how the parts are wired, a key of the arrangement registry
    (``models.decoder.register_arrangement``); ``pre_norm`` is
    ``x += mixer(norm(x)); x += ff(norm(x))`` (src/model/cpu_llama.cpp:62-98).  A block whose
    arrangement has no feed-forward, or no second norm, leaves those fields ``None``.
    """

    arrangement: str
    mixer_norm: PartSpec
    mixer: PartSpec
    feed_forward_norm: Optional[PartSpec] = None
    feed_forward: Optional[PartSpec] = None


@dataclasses.dataclass(frozen=True)
class ScheduleEntry:
    """One executed layer.  ``block`` indexes ``ModelSpec.blocks``.

    ``cache_from`` is the index of an earlier schedule entry whose key/value
    cache (or state) this entry reads instead of owning one; ``None`` means the
    entry owns its cache.
    """

    block: int
    cache_from: Optional[int] = None


@dataclasses.dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    blocks: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    lm_head: PartSpec

    def validate(self) -> None:
        if not self.blocks or not self.schedule:
            raise ValueError("a model needs at least one block and one schedule entry")
        for index, entry in enumerate(self.schedule):
            if not 0 <= entry.block < len(self.blocks):
                raise ValueError(f"schedule entry {index} names block {entry.block}, "
                                 f"but there are {len(self.blocks)} blocks")
            if entry.cache_from is not None:
                if not 0 <= entry.cache_from < index:
                    raise ValueError(f"schedule entry {index} reads the cache of entry "
                                     f"{entry.cache_from}, which does not run before it")
                if self.schedule[entry.cache_from].cache_from is not None:
                    raise ValueError(f"schedule entry {index} reads the cache of entry "
                                     f"{entry.cache_from}, which owns none")
