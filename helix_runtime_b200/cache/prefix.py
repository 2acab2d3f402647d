"""Prefix index: prompts that begin alike share the pages of their common beginning.

The index maps (namespace, exact tokens of a page-aligned prefix) to an *anchor* of the cache
manager that keeps those pages alive.  It follows the reference's ``PagedPrefixCache``
(src/kv_cache/prefix.cpp:96-117, 196-206, 365-409) and the rules its engine applies around it
(src/runtime/cpu_engine.cpp:30-36, 136-160, 323-331):

* keys are a namespace plus the exact token ids; an incremental FNV-1a digest per aligned
  length finds candidates (every aligned length of a published prefix is a key, so a later
  prompt may share only the first pages of it), a full comparison of the tokens confirms a hit;
  when the cache has a group with a window, an anchor holds only the pages that window reaches
  from the END of the prefix, and when the model keeps per-request state, the state at its
  end, so only the prefix's full length is a key: a later prompt that goes on from it (the
  next turn of a conversation) shares it, one that departs earlier does not;
* a request reuses at most ``floor((P - 1) / page) * page`` tokens of a prompt of ``P``
  tokens: keys and values are cached, logits are not, so at least one prompt token must run;
* a prefix is published when the request's LAST prompt portion has succeeded, and only its
  longest aligned prefix ``floor(P / page) * page``;
* entries are kept in least-recently-used order under two budgets (entries, page references);
  the engine also evicts from the cold end when pages run out, before any request has to wait.

Positions are absolute in the cache (keys are stored after the rotary encoding), so a shared
prefix always starts at position 0.
"""
from __future__ import annotations

import dataclasses
from collections import OrderedDict
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from .manager import CacheManager

FNV_OFFSET = 0xCBF29CE484222325
FNV_PRIME = 0x100000001B3
MASK64 = (1 << 64) - 1


def fnv1a_step(digest: int, token: int) -> int:
    """One token (as four little-endian bytes) into a 64-bit FNV-1a digest."""
    for shift in (0, 8, 16, 24):
        digest ^= (token >> shift) & 0xFF
        digest = (digest * FNV_PRIME) & MASK64
    return digest


def aligned_digests(tokens: Sequence[int], page_size: int, limit: int) -> List[Tuple[int, int]]:
    """``(length, digest)`` for every page-aligned prefix length up to ``limit``."""
    out = []
    digest = FNV_OFFSET
    for index in range(min(limit, len(tokens))):
        digest = fnv1a_step(digest, int(tokens[index]))
        if (index + 1) % page_size == 0:
            out.append((index + 1, digest))
    return out


@dataclasses.dataclass
class PrefixEntry:
    anchor: Hashable
    namespace: str
    tokens: Tuple[int, ...]
    pages: int
    keys: Tuple[Tuple[str, int, int], ...] = ()
    hits: int = 0


@dataclasses.dataclass(frozen=True)
class PrefixMatch:
    anchor: Hashable
    tokens: int           # how many tokens of the prompt the request may adopt


class PrefixIndex:
    def __init__(self, cache: CacheManager, maximum_entries: int,
                 maximum_page_references: Optional[int] = None) -> None:
        if maximum_entries <= 0:
            raise ValueError("maximum_entries must be positive")
        self.cache = cache
        self.page_size = cache.page_size
        self.maximum_entries = int(maximum_entries)
        # an entry's pages are counted as its prefix's length in pages, which is what it holds
        # of every group that keeps all keys (a windowed group holds a few pages per entry)
        pools = [group.pool.num_pages for group in cache.groups if group.need.window is None] \
            or [group.pool.num_pages for group in cache.groups]
        smallest_pool = min(pools)
        self.maximum_page_references = int(maximum_page_references
                                           if maximum_page_references is not None
                                           else smallest_pool // 2)
        # anchor -> entry, coldest first
        self._entries: "OrderedDict[Hashable, PrefixEntry]" = OrderedDict()
        # (namespace, length, digest) -> anchors with that key (collisions are possible)
        self._by_key: Dict[Tuple[str, int, int], List[Hashable]] = {}
        self._next_anchor = 0
        self.stats = {"lookups": 0, "hits": 0, "reused_tokens": 0, "published": 0,
                      "not_kept": 0, "evicted": 0, "evicted_under_pressure": 0}

    def __len__(self) -> int:
        return len(self._entries)

    @property
    def page_references(self) -> int:
        return sum(entry.pages for entry in self._entries.values())

    def reuse_bound(self, prompt_tokens: int) -> int:
        """The most tokens of a prompt that may come from the index."""
        return max(0, (prompt_tokens - 1) // self.page_size) * self.page_size

    # ------------------------------------------------------------------- lookup

    def lookup(self, namespace: Optional[str], tokens: Sequence[int]) -> Optional[PrefixMatch]:
        """The longest published prefix of ``tokens`` within the reuse bound, or None.  A hit
        makes the entry the most recently used."""
        if namespace is None or not self._entries:
            return None
        self.stats["lookups"] += 1
        bound = self.reuse_bound(len(tokens))
        for length, digest in reversed(aligned_digests(tokens, self.page_size, bound)):
            for anchor in self._by_key.get((namespace, length, digest), ()):
                entry = self._entries[anchor]
                if entry.tokens[:length] == tuple(int(t) for t in tokens[:length]):
                    self._entries.move_to_end(anchor)
                    entry.hits += 1
                    self.stats["hits"] += 1
                    self.stats["reused_tokens"] += length
                    return PrefixMatch(anchor, length)
        return None

    # ------------------------------------------------------------------ publish

    def publish(self, namespace: Optional[str], request: Hashable,
                prompt: Sequence[int]) -> Optional[Hashable]:
        """Keep the longest aligned prefix of ``prompt`` (whose keys and values ``request``
        has published in the cache) for later requests.  Returns the anchor, or None when
        there is nothing to keep, it is already kept, or it cannot fit the budgets."""
        if namespace is None:
            return None
        length = (len(prompt) // self.page_size) * self.page_size
        if length == 0 or self.cache.length(request) < length:
            return None
        pages = length // self.page_size
        if pages > self.maximum_page_references:
            return None
        tokens = tuple(int(t) for t in prompt[:length])
        digests = aligned_digests(tokens, self.page_size, length)
        for anchor in self._by_key.get((namespace, length, digests[-1][1]), ()):
            if self._entries[anchor].tokens[:length] == tokens:
                self._entries.move_to_end(anchor)      # this prefix (or a longer one) is kept
                return None
        while self._entries and (len(self._entries) >= self.maximum_entries or
                                 self.page_references + pages > self.maximum_page_references):
            self._evict_coldest()
        anchor = ("prefix", self._next_anchor)
        try:
            self.cache.hold(anchor, request, length)
        except ValueError:
            # a windowed group has given back pages the prefix's end still reads, or no
            # state was kept at the prefix's end
            self.stats["not_kept"] += 1
            return None
        self._next_anchor += 1
        # every aligned length of the prefix is a key: a later prompt may share only the
        # first pages of it; with a windowed group only all of it can be shared
        if self.cache.shares_whole_prefixes_only:
            digests = digests[-1:]
        keys = tuple((namespace, part, digest) for part, digest in digests)
        self._entries[anchor] = PrefixEntry(anchor, namespace, tokens, pages, keys)
        for key in keys:
            self._by_key.setdefault(key, []).append(anchor)
        self.stats["published"] += 1
        return anchor

    # ----------------------------------------------------------------- eviction

    def _evict_coldest(self) -> int:
        anchor, entry = self._entries.popitem(last=False)
        for key in entry.keys:
            self._by_key[key].remove(anchor)
            if not self._by_key[key]:
                del self._by_key[key]
        self.stats["evicted"] += 1
        return self.cache.drop(anchor)

    def evict_for_pressure(self) -> bool:
        """Pages ran out: drop the coldest entry.  True when an entry was dropped (pages come
        free only when no live request shares them)."""
        if not self._entries:
            return False
        self._evict_coldest()
        self.stats["evicted_under_pressure"] += 1
        return True

    def clear(self) -> None:
        while self._entries:
            self._evict_coldest()
