"""The cache manager: paged keys and values with a block table per request, and state slots.

Layers with the same needs (``kv_heads``, ``head_dim``, ``window``) form a *group*;
each group has its own pool of pages, its own key/value storage and its own block
tables, so a model whose layers differ (all keys here, a window of them there) gives
every kind of layer pages of the right shape and gives a window's pages back as soon
as the window has passed them.  The reference has one geometry for all layers
(src/kv_cache/paged.cpp:100-104, src/model/cuda_llama.cpp:147-154); groups are this
engine's own.

A page id is valid in every layer of its group (as in the reference, where a block
spans all layers).  Storage of one group is ``[layer, key|value, page, kv_head, ...]``; the
last two axes hold ``page_size x head_dim`` elements in the kernels' chunked order
``[head_dim / c, slot, c]`` (``c`` elements = 16 bytes), so that everything a (page, head)
holds is one contiguous block.

Pages are reserved before a step (:meth:`CacheManager.extend`) and a request's
length is published after it (:meth:`CacheManager.commit`), which is the reference's
transaction boundary (src/runtime/cpu_engine.cpp:191, 207, 235).

Deferred reclamation.  A request may end while a step that still reads or writes its pages
is queued on the device (cancelled in flight; retired by the step before the one queued
ahead).  ``release(request, after=step)`` then PARKS its pages and its slot behind that
step's sequence number; they return to the ring, in the order they were parked, when the
engine reports that step complete (:meth:`CacheManager.settle`), and only then can they
reach another request.  The reference built the same rule into an allocator of its own (a
free is held until a completion is ready, src/memory/deferred_allocator.cpp:43-70, an event
on the releasing stream, src/memory/stream_ordered_allocator.cpp:15-31) and never wired it to
its cache; here the unit is the page and the completion is the step.  Next to the pages
every request owns one *state slot*: a row in each per-layer state tensor that a
mixer asked for (fixed size, zeroed at admission), and a row in the block tables.
"""
from __future__ import annotations

import dataclasses
from collections import deque
from typing import Deque, Dict, Hashable, List, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch

from .pages import OutOfPages, PagePool


@dataclasses.dataclass(frozen=True)
class KvNeed:
    """What an attention-like mixer needs of the cache."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None     # None: every earlier key stays live


@dataclasses.dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size that a mixer keeps between steps."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class CacheGroup:
    def __init__(self, index: int, need: KvNeed, entries: List[int], num_pages: int,
                 page_size: int, max_requests: int, max_pages_per_request: int,
                 dtype: torch.dtype, device: torch.device, poison: bool) -> None:
        self.index = index
        self.need = need
        self.entries = entries                      # schedule entries that own a layer here
        self.pool = PagePool(num_pages)
        self.page_size = page_size
        self.poison = poison
        shape = (len(entries), 2, num_pages, need.kv_heads, page_size, need.head_dim)
        if poison:
            self.storage = torch.full(shape, float("nan"), dtype=dtype, device=device)
        else:
            self.storage = torch.zeros(shape, dtype=dtype, device=device)
        self.host_tables = np.full((max_requests, max_pages_per_request), -1, dtype=np.int32)
        # uploads go through a pinned copy, so that they queue behind the step in flight
        # instead of waiting for it; the event says when the pinned copy may be rewritten
        pinned = device.type == "cuda"
        self._staging = torch.full((max_requests, max_pages_per_request), -1, dtype=torch.int32,
                                   pin_memory=pinned)
        self._staged = torch.cuda.Event() if pinned else None
        self.device_tables = torch.full((max_requests, max_pages_per_request), -1,
                                        dtype=torch.int32, device=device)
        self.dirty = False

    def upload_tables(self) -> None:
        if self._staged is not None:
            self._staged.synchronize()       # the last upload has left the pinned copy
        self._staging.numpy()[:] = self.host_tables
        self.device_tables.copy_(self._staging, non_blocking=True)
        if self._staged is not None:
            self._staged.record()
        self.dirty = False

    @property
    def bytes_per_token(self) -> int:
        return (len(self.entries) * 2 * self.need.kv_heads * self.need.head_dim
                * self.storage.element_size())


@dataclasses.dataclass
class RequestCache:
    slot: int
    length: int = 0                                  # tokens whose keys/values are published
    reserved: int = 0                                # tokens the tables have pages for
    tables: List[List[int]] = dataclasses.field(default_factory=list)   # per group, -1 = gone
    first_live: List[int] = dataclasses.field(default_factory=list)     # per group
    # per-request state as it stood after `kept_state_length` tokens: copies, one per entry
    kept_state_length: int = -1
    kept_state: Optional[Dict[int, torch.Tensor]] = None


@dataclasses.dataclass
class Anchor:
    """Pages (per group, by page index; -1 where a window had passed) and, for models with
    per-request state, the state at the end of a prefix of ``tokens`` tokens."""
    tokens: int
    pages: List[List[int]]
    state: Optional[Dict[int, torch.Tensor]] = None


class CacheManager:
    def __init__(self, kv_needs: Mapping[int, KvNeed], state_needs: Mapping[int, StateNeed],
                 page_size: int, num_pages: int, max_requests: int, max_positions: int,
                 dtype: torch.dtype, device: torch.device, poison: bool = False,
                 window_slack_pages: int = 0,
                 window_pages: Optional[Mapping[int, int]] = None) -> None:
        if page_size <= 0 or max_requests <= 0 or max_positions <= 0:
            raise ValueError("page_size, max_requests and max_positions must be positive")
        if window_slack_pages < 0:
            raise ValueError("window_slack_pages must not be negative")
        self.page_size = int(page_size)
        # Pages a windowed group keeps behind its window before it gives them back.  A prefix
        # is kept for later requests at the last page boundary of a prompt, up to a page
        # short of where its request stands by then: with one page of slack the keys that the
        # window of that boundary reaches back to are still there.
        self.window_slack_pages = int(window_slack_pages)
        self.max_requests = int(max_requests)
        self.max_positions = int(max_positions)
        self.max_pages_per_request = -(-self.max_positions // self.page_size)
        self.dtype = dtype
        self.device = device
        self.groups: List[CacheGroup] = []
        self._entry_place: Dict[int, Tuple[int, int]] = {}
        by_need: Dict[KvNeed, List[int]] = {}
        for entry in sorted(kv_needs):
            by_need.setdefault(kv_needs[entry], []).append(entry)
        # ``num_pages`` is every group's pool unless ``window_pages`` gives the groups of a
        # window (by its length) a pool of their own size: a request never holds more of such
        # a group than its window, the page being filled and the portion it is fed.
        window_pages = dict(window_pages or {})
        unknown = set(window_pages) - {need.window for need in by_need}
        if unknown:
            raise ValueError(f"window_pages names windows no layer has: {sorted(unknown)}")
        for need, entries in by_need.items():
            pages = window_pages.get(need.window, num_pages) if need.window is not None \
                else num_pages
            if pages <= 0:
                raise ValueError("a pool needs at least one page")
            group = CacheGroup(len(self.groups), need, entries, pages, self.page_size,
                               self.max_requests, self.max_pages_per_request, dtype, device, poison)
            for layer, entry in enumerate(entries):
                self._entry_place[entry] = (group.index, layer)
            self.groups.append(group)
        self.states: Dict[int, torch.Tensor] = {
            entry: torch.zeros((self.max_requests, *need.shape), dtype=need.dtype, device=device)
            for entry, need in state_needs.items()}
        self._free_slots: Deque[int] = deque(range(self.max_requests))
        self._requests: Dict[Hashable, RequestCache] = {}
        # page lists held without a request (published prefixes): per anchor, per group
        self._anchors: Dict[Hashable, Anchor] = {}
        # what was given up while a step still used it: (step, slot or None, pages per group),
        # oldest first
        self._parked: Deque[Tuple[int, Optional[int], List[List[int]]]] = deque()
        self.settled_step = -1

    # ------------------------------------------------------------------ lookups

    def owns_pages(self, entry: int) -> bool:
        """Whether this schedule entry has key/value storage here."""
        return entry in self._entry_place

    def group_of(self, entry: int) -> CacheGroup:
        return self.groups[self._entry_place[entry][0]]

    def layer_storage(self, entry: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Key and value storage of one schedule entry: ``[page, kv_head, page_size, head_dim]`` in
        shape, the last two axes in the kernels' chunked order (see the module's docstring)."""
        group_index, layer = self._entry_place[entry]
        storage = self.groups[group_index].storage
        return storage[layer, 0], storage[layer, 1]

    def state(self, entry: int) -> torch.Tensor:
        return self.states[entry]

    def has(self, request: Hashable) -> bool:
        return request in self._requests

    def slot(self, request: Hashable) -> int:
        return self._requests[request].slot

    def length(self, request: Hashable) -> int:
        return self._requests[request].length

    def reserved(self, request: Hashable) -> int:
        """Positions the request has pages for: its length plus what steps in flight add."""
        return self._requests[request].reserved

    def live_requests(self) -> List[Hashable]:
        return list(self._requests)

    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def free_pages(self) -> List[int]:
        return [group.pool.free_pages for group in self.groups]

    def bytes_per_token(self) -> int:
        return sum(group.bytes_per_token for group in self.groups)

    # --------------------------------------------------------------- page maths

    def pages_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    def pages_needed_alone(self, rows: int) -> List[int]:
        """Pages of each group that a request of ``rows`` cache rows must be able to hold at
        once to run to its end alone, fed in portions as small as the pool demands.  A group
        that keeps every key needs all its pages; a windowed group gives pages back as its
        window passes them and never holds more than the window and the page being filled."""
        needed = []
        for group in self.groups:
            window = group.need.window
            live = rows if window is None else \
                min(rows, window + (1 + self.window_slack_pages) * self.page_size)
            needed.append(self.pages_for(live))
        return needed

    def first_page_seen(self, group: CacheGroup, length: int) -> int:
        """Index of the first page that the query at position ``length`` still reads in
        ``group``: 0 without a window."""
        window = group.need.window
        if window is None:
            return 0
        return max(0, length - window + 1) // self.page_size

    def pages_to_extend(self, request: Hashable, new_length: int) -> List[int]:
        """Pages each group must add so that positions ``[0, new_length)`` have a place."""
        record = self._requests[request]
        return [max(0, self.pages_for(new_length) - len(table)) for table in record.tables]

    def max_extend(self, request: Hashable, desired: int,
                   available: Optional[Sequence[int]] = None) -> int:
        """The most tokens (``<= desired``) that can be appended with ``available`` free pages
        per group (default: what the pools hold now)."""
        record = self._requests[request]
        if available is None:
            available = self.free_pages()
        base = record.reserved
        room = min(self.max_positions - base, desired)
        best = max(room, 0)
        for table, free in zip(record.tables, available):
            tokens_with_pages = (len(table) + free) * self.page_size
            best = min(best, max(0, tokens_with_pages - base))
        return best

    def max_extend_new(self, desired: int, available: Optional[Sequence[int]] = None) -> int:
        """Same for a request that is not admitted yet (no pages, length 0)."""
        if available is None:
            available = self.free_pages()
        best = min(desired, self.max_positions)
        for free in available:
            best = min(best, free * self.page_size)
        return max(best, 0)

    # ------------------------------------------------------------- life of a request

    def admit(self, request: Hashable) -> int:
        """Give the request a state slot (zeroed) and empty block tables."""
        if request in self._requests:
            raise KeyError(f"request {request!r} is already admitted")
        if not self._free_slots:
            raise OutOfPages("no state slot is free")
        slot = self._free_slots.popleft()
        for tensor in self.states.values():
            tensor[slot].zero_()
        for group in self.groups:
            group.host_tables[slot, :] = -1
            group.dirty = True
        self._requests[request] = RequestCache(
            slot=slot, tables=[[] for _ in self.groups], first_live=[0 for _ in self.groups])
        return slot

    def extend(self, request: Hashable, new_length: int) -> List[int]:
        """Reserve pages for positions up to ``new_length`` in every group, or raise
        :class:`OutOfPages` and change nothing.  Returns the pages added per group."""
        record = self._requests[request]
        if new_length > self.max_positions:
            raise ValueError(f"length {new_length} exceeds max_positions {self.max_positions}")
        if new_length < record.length:
            raise ValueError("a request's cache never shrinks")
        needed = self.pages_to_extend(request, new_length)
        for group, count in zip(self.groups, needed):
            if count > group.pool.free_pages:
                raise OutOfPages(f"group {group.index}: {count} pages needed, "
                                 f"{group.pool.free_pages} free")
        for group, table, count in zip(self.groups, record.tables, needed):
            if count == 0:
                continue
            pages = group.pool.allocate(count)
            start = len(table)
            table.extend(pages)
            group.host_tables[record.slot, start:start + count] = pages
            group.dirty = True
        record.reserved = max(record.reserved, new_length)
        return needed

    def commit(self, request: Hashable, new_length: int) -> None:
        """Publish the length after a step that succeeded; give back pages a window passed."""
        record = self._requests[request]
        if new_length < record.length or new_length > record.reserved:
            raise ValueError(f"cannot publish length {new_length}: published {record.length}, "
                             f"reserved {record.reserved}")
        record.length = new_length
        for index, group in enumerate(self.groups):
            window = group.need.window
            if window is None:
                continue
            # the next query sits at position new_length and reads keys >= new_length-window+1
            dead_pages = max(0, self.first_page_seen(group, new_length) - self.window_slack_pages)
            table = record.tables[index]
            first = record.first_live[index]
            if dead_pages > first:
                gone = [table[i] for i in range(first, dead_pages)]
                self._give_back(group, gone)
                for i in range(first, dead_pages):
                    table[i] = -1
                group.host_tables[record.slot, first:dead_pages] = -1
                group.dirty = True
                record.first_live[index] = dead_pages

    def rollback(self, request: Hashable, keep_length: Optional[int] = None,
                 after: Optional[int] = None) -> None:
        """Give back pages reserved beyond the published length (a step that failed), or
        beyond ``keep_length`` when an earlier step that reserved up to there is still in
        flight.  ``after``: a step on the device that may still write them (see
        :meth:`release`)."""
        record = self._requests[request]
        target = record.length if keep_length is None else keep_length
        if not record.length <= target <= record.reserved:
            raise ValueError(f"cannot roll back to {target}: published {record.length}, "
                             f"reserved {record.reserved}")
        keep = self.pages_for(target)
        parked: List[List[int]] = []
        for index, group in enumerate(self.groups):
            table = record.tables[index]
            extra: List[int] = []
            if len(table) > keep:
                extra = [page for page in table[keep:] if page >= 0]
                group.host_tables[record.slot, keep:len(table)] = -1
                del table[keep:]
                group.dirty = True
            parked.append(extra)
        if after is not None and after > self.settled_step and any(parked):
            self._parked.append((after, None, parked))
        else:
            for group, pages in zip(self.groups, parked):
                self._give_back(group, pages)
        record.reserved = target

    def release(self, request: Hashable, after: Optional[int] = None) -> int:
        """The request is over: give back its pages (in table order) and its slot.  ``after``:
        the sequence number of a step on the device that may still touch them; pages and slot
        are then parked until :meth:`settle` hears that step is complete.  Returns the pages
        that became free now."""
        record = self._requests.pop(request)
        held = [[page for page in record.tables[index] if page >= 0]
                for index in range(len(self.groups))]
        for group in self.groups:
            group.host_tables[record.slot, :] = -1
            group.dirty = True
        if after is not None and after > self.settled_step:
            self._parked.append((after, record.slot, held))
            return 0
        self._free_slots.append(record.slot)
        return sum(self._give_back(group, pages) for group, pages in zip(self.groups, held))

    def settle(self, step: int) -> int:
        """Every step up to ``step`` has completed on the device: what was parked behind them
        goes back, oldest first.  Returns the pages that became free."""
        self.settled_step = max(self.settled_step, step)
        freed = 0
        while self._parked and self._parked[0][0] <= self.settled_step:
            _, slot, held = self._parked.popleft()
            if slot is not None:
                self._free_slots.append(slot)
            freed += sum(self._give_back(group, pages) for group, pages in zip(self.groups, held))
        return freed

    @property
    def parked_pages(self) -> int:
        """Pages (summed over groups) that wait for a step to complete."""
        return sum(len(pages) for _, _, held in self._parked for pages in held)

    def _shared_pages(self, parent: RequestCache, tokens: int) -> List[List[int]]:
        """The pages of ``parent`` that a request standing at ``tokens`` reads, per group, by
        page index (-1 where a window has passed: nobody reads there again).  Raises when a
        page that is still read has been given back already."""
        count = tokens // self.page_size
        shared = []
        for index, group in enumerate(self.groups):
            first = self.first_page_seen(group, tokens)
            if parent.first_live[index] > first:
                raise ValueError(
                    f"group {group.index}: the source has given back pages that a request at "
                    f"{tokens} tokens still reads (window {group.need.window})")
            shared.append([-1] * first + list(parent.tables[index][first:count]))
        return shared

    def _state_at(self, parent: RequestCache, tokens: int) -> Optional[Dict[int, torch.Tensor]]:
        """The kept state of ``parent`` if it is the state after exactly ``tokens`` tokens."""
        if not self.states:
            return None
        if parent.kept_state is None or parent.kept_state_length != tokens:
            raise ValueError(f"no state was kept after {tokens} tokens "
                             f"(kept after {parent.kept_state_length})")
        return parent.kept_state

    def _admit_with(self, request: Hashable, tokens: int, shared: List[List[int]],
                    state: Optional[Dict[int, torch.Tensor]] = None) -> int:
        slot = self.admit(request)
        record = self._requests[request]
        if state is not None:
            for entry, tensor in self.states.items():
                tensor[slot].copy_(state[entry])
            record.kept_state_length, record.kept_state = tokens, state
        count = tokens // self.page_size
        for index, group in enumerate(self.groups):
            pages = shared[index][:count]
            group.pool.share([page for page in pages if page >= 0])
            record.tables[index] = list(pages)
            record.first_live[index] = next((i for i, page in enumerate(pages) if page >= 0), count)
            group.host_tables[slot, :count] = pages
            group.dirty = True
        record.length = tokens
        record.reserved = tokens
        return slot

    def fork(self, source: Hashable, request: Hashable, tokens: int) -> int:
        """Admit ``request`` sharing the first ``tokens`` positions of ``source``.

        Only whole pages are shared, so nothing is ever copied on write
        (src/kv_cache/paged.cpp:535-620).  A group with a window shares the pages its window
        still reaches from ``tokens``; they must not have been given back yet.  With
        per-request state the source must have kept its state after exactly ``tokens``."""
        if tokens <= 0 or tokens % self.page_size != 0:
            raise ValueError("a shared prefix must be a positive multiple of the page size")
        parent = self._requests[source]
        if tokens > parent.length:
            raise ValueError("cannot share more than the source has published")
        return self._admit_with(request, tokens, self._shared_pages(parent, tokens),
                                self._state_at(parent, tokens))

    # ------------------------------------------------------------------ anchors
    #
    # An anchor keeps the whole pages of a prefix alive after the request that computed them
    # has gone (src/kv_cache/prefix.cpp holds block references the same way).  It has no
    # state slot and no block-table row: it is only a holder of pages.

    @property
    def shares_whole_prefixes_only(self) -> bool:
        """With a windowed group an anchor holds the pages its window reaches from the END of
        the prefix, and with per-request state the state at its end, so a request can adopt
        all of the prefix or none of it; otherwise any number of its leading pages."""
        return bool(self.states) or any(group.need.window is not None for group in self.groups)

    # Per-request state is not in pages: what a later request needs of a prefix is the state
    # as it stood at the prefix's end.  The engine copies it there (in stream order behind the
    # step that reaches that length, before the next step changes it) and hands the copy to
    # the request's record once the step has succeeded.

    def snapshot_state(self, request: Hashable) -> Dict[int, torch.Tensor]:
        """Copies of the request's state rows, queued on the current stream."""
        slot = self._requests[request].slot
        return {entry: tensor[slot].clone() for entry, tensor in self.states.items()}

    def keep_state(self, request: Hashable, tokens: int, snapshot: Dict[int, torch.Tensor]) -> None:
        """``snapshot`` is the request's state after ``tokens`` tokens."""
        record = self._requests[request]
        if sorted(snapshot) != sorted(self.states):
            raise ValueError("a state snapshot has one tensor per state entry")
        record.kept_state_length, record.kept_state = int(tokens), snapshot

    def hold(self, anchor: Hashable, source: Hashable, tokens: int) -> int:
        """Keep the first ``tokens`` positions (whole pages) of ``source`` under ``anchor``;
        returns the page references it now holds, summed over groups.  Raises ValueError
        when a windowed group of the source has already given back pages it would need, or
        when the model has per-request state and none was kept after ``tokens``."""
        if anchor in self._anchors:
            raise KeyError(f"anchor {anchor!r} exists")
        if tokens <= 0 or tokens % self.page_size != 0:
            raise ValueError("a shared prefix must be a positive multiple of the page size")
        parent = self._requests[source]
        if tokens > parent.length:
            raise ValueError("cannot share more than the source has published")
        held = self._shared_pages(parent, tokens)
        state = self._state_at(parent, tokens)
        for group, pages in zip(self.groups, held):
            group.pool.share([page for page in pages if page >= 0])
        self._anchors[anchor] = Anchor(tokens, held, state)
        return sum(1 for pages in held for page in pages if page >= 0)

    def adopt(self, request: Hashable, anchor: Hashable, tokens: Optional[int] = None) -> int:
        """Admit ``request`` with the first ``tokens`` positions (default: all) of ``anchor``
        already in its cache; returns its slot."""
        kept = self._anchors[anchor]
        tokens = kept.tokens if tokens is None else tokens
        if tokens <= 0 or tokens % self.page_size != 0 or tokens > kept.tokens:
            raise ValueError("a request adopts a positive number of whole pages of the anchor")
        if tokens != kept.tokens and self.shares_whole_prefixes_only:
            raise ValueError("with a windowed group or per-request state a request adopts all "
                             "of an anchor or none")
        return self._admit_with(request, tokens, kept.pages, kept.state)

    def drop(self, anchor: Hashable) -> int:
        """Forget the anchor; returns the pages that became free."""
        kept = self._anchors.pop(anchor)
        return sum(self._give_back(group, [page for page in pages if page >= 0])
                   for group, pages in zip(self.groups, kept.pages))

    def anchor_pages(self) -> int:
        """Pages (per group, summed) that anchors hold references to."""
        return sum(1 for kept in self._anchors.values() for pages in kept.pages
                   for page in pages if page >= 0)

    def _give_back(self, group: CacheGroup, pages: List[int]) -> int:
        if not pages:
            return 0
        freed = group.pool.release(pages)
        if group.poison and freed:
            index = torch.tensor(group.pool.last_freed(freed), dtype=torch.long,
                                 device=group.storage.device)
            group.storage[:, :, index] = float("nan")
        return freed

    # ------------------------------------------------------------------- device

    def sync_tables(self) -> None:
        """Copy block tables that changed since the last step to the device."""
        for group in self.groups:
            if group.dirty:
                group.upload_tables()

    # -------------------------------------------------------------------- audit

    def check(self) -> None:
        """No page lost, held twice by mistake, or freed twice; no slot lost."""
        slots = [record.slot for record in self._requests.values()] + \
            [slot for _, slot, _ in self._parked if slot is not None]
        assert len(slots) == len(set(slots)), "a state slot is held twice"
        assert sorted(slots + list(self._free_slots)) == list(range(self.max_requests)), \
            "a state slot is lost"
        for index, group in enumerate(self.groups):
            group.pool.check()
            holders = [0] * group.pool.num_pages
            for record in self._requests.values():
                table = record.tables[index]
                live = [page for page in table if page >= 0]
                assert len(live) == len(set(live)), "a request holds a page twice"
                for page in live:
                    holders[page] += 1
                assert len(table) >= self.pages_for(record.length), "published tokens lack a page"
                row = group.host_tables[record.slot]
                assert list(row[:len(table)]) == table, "host block table out of date"
                assert (row[len(table):] == -1).all(), "stale block table entries"
            for anchor in self._anchors.values():
                kept = [page for page in anchor.pages[index] if page >= 0]
                assert len(kept) == len(set(kept)), "an anchor holds a page twice"
                for page in kept:
                    holders[page] += 1
            for _, _, held in self._parked:
                for page in held[index]:
                    holders[page] += 1
            for page in range(group.pool.num_pages):
                assert holders[page] == group.pool.refcount(page), \
                    f"group {index} page {page}: {holders[page]} holders, " \
                    f"refcount {group.pool.refcount(page)}"

    def stats(self) -> Dict[str, object]:
        return {
            "requests": len(self._requests),
            "free_slots": len(self._free_slots),
            "anchors": len(self._anchors),
            "anchor_pages": self.anchor_pages(),
            "parked_pages": self.parked_pages,
            "groups": [{
                "window": group.need.window,
                "layers": len(group.entries),
                "pages": group.pool.num_pages,
                "free_pages": group.pool.free_pages,
                "peak_pages_in_use": group.pool.peak_in_use,
                "allocations": group.pool.allocation_count,
                "reuses": group.pool.reuse_count,
            } for group in self.groups],
        }
