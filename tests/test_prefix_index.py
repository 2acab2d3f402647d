"""The prefix index on the CPU: what is found, what is kept and what is dropped, and that pages
held by kept prefixes are never lost, held twice by mistake or freed twice
(rules: src/kv_cache/prefix.cpp:96-117, 196-206, 365-409; src/runtime/cpu_engine.cpp:30-36,
136-160, 323-331)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helix_runtime_b200.cache import CacheManager, KvNeed, PrefixIndex, StateNeed
from helix_runtime_b200.cache import prefix as prefix_module
from helix_runtime_b200.engine import FifoScheduler, SchedulerConfig, WorkCompletion, WorkKind

CPU = torch.device("cpu")
PAGE = 4


def manager(num_pages=32, max_requests=4, window=None, states=None, slack=0):
    needs = {0: KvNeed(2, 8), 1: KvNeed(2, 8)}
    if window is not None:
        needs[2] = KvNeed(2, 8, window=window)
    return CacheManager(needs, states or {}, PAGE, num_pages, max_requests, 256, torch.float32, CPU,
                        window_slack_pages=slack)


def run_prompt(cache, request, tokens, adopt=None):
    """What the engine does for a prompt: admit (or adopt), reserve, publish the length."""
    if adopt is None:
        cache.admit(request)
    else:
        cache.adopt(request, adopt.anchor, adopt.tokens)
    cache.extend(request, len(tokens))
    cache.commit(request, len(tokens))


def test_longest_aligned_prefix_is_found_and_one_token_always_runs():
    cache = manager()
    index = PrefixIndex(cache, maximum_entries=8)
    prompt = list(range(100, 114))                       # 14 tokens: 3 whole pages
    run_prompt(cache, "a", prompt)
    anchor = index.publish("ns", "a", prompt)
    assert anchor is not None and len(index) == 1 and index.page_references == 3
    cache.release("a")                                   # the pages outlive the request
    cache.check()
    assert cache.groups[0].pool.pages_in_use == 3

    # the same prompt again: 12 tokens are kept, and 12 <= floor(13 / 4) * 4 may be reused
    match = index.lookup("ns", prompt)
    assert match is not None and match.tokens == 12
    # a prompt that IS the kept prefix must still run one token: only 8 may be reused
    assert index.lookup("ns", prompt[:12]).tokens == 8
    assert index.reuse_bound(12) == 8 and index.reuse_bound(13) == 12 and index.reuse_bound(1) == 0
    # a prompt that shares only the first 9 tokens adopts the first two pages of the entry
    other = prompt[:9] + [7, 7, 7, 7, 7]
    assert index.lookup("ns", other).tokens == 8
    # nothing in common, another namespace, no namespace
    assert index.lookup("ns", [1, 2, 3, 4, 5, 6]) is None
    assert index.lookup("elsewhere", prompt) is None
    assert index.lookup(None, prompt) is None
    assert index.publish(None, "a", prompt) is None

    run_prompt(cache, "b", other, adopt=index.lookup("ns", other))
    assert cache.length("b") == len(other)
    pool = cache.groups[0].pool
    shared = cache._requests["b"].tables[0][:2]
    assert all(pool.refcount(page) == 2 for page in shared)
    cache.check()
    cache.release("b")
    cache.check()
    assert pool.pages_in_use == 3


def test_publishing_twice_keeps_one_entry_and_a_short_prompt_keeps_nothing():
    cache = manager()
    index = PrefixIndex(cache, maximum_entries=8)
    prompt = list(range(20))
    run_prompt(cache, "a", prompt)
    assert index.publish("ns", "a", prompt) is not None
    assert index.publish("ns", "a", prompt) is None
    assert index.publish("ns", "a", prompt[:17]) is None      # a part of what is kept already
    assert len(index) == 1
    run_prompt(cache, "tiny", [1, 2, 3])
    assert index.publish("ns", "tiny", [1, 2, 3]) is None     # less than a page
    cache.admit("unrun")
    assert index.publish("ns", "unrun", prompt) is None       # its keys are not in the cache
    cache.check()


def test_least_recently_used_entries_go_first_under_both_budgets():
    cache = manager(num_pages=64)
    index = PrefixIndex(cache, maximum_entries=3, maximum_page_references=10)
    prompts = {name: [base + i for i in range(9)] for name, base in
               (("a", 100), ("b", 200), ("c", 300), ("d", 400))}       # 2 pages each
    for name in ("a", "b", "c"):
        run_prompt(cache, name, prompts[name])
        index.publish("ns", name, prompts[name])
        cache.release(name)
    assert index.lookup("ns", prompts["a"]) is not None                # a is warm again
    run_prompt(cache, "d", prompts["d"])
    index.publish("ns", "d", prompts["d"])                             # a fourth entry: b goes
    cache.release("d")
    assert index.lookup("ns", prompts["b"]) is None
    assert all(index.lookup("ns", prompts[name]) is not None for name in ("a", "c", "d"))
    assert index.stats["evicted"] == 1
    # a prefix of 9 pages fits the page budget of 10 only alone
    long_prompt = list(range(1000, 1037))
    run_prompt(cache, "long", long_prompt)
    index.publish("ns", "long", long_prompt)
    assert len(index) == 1 and index.page_references == 9
    # and one of 11 pages is not kept at all
    longer = list(range(2000, 2045))
    run_prompt(cache, "longer", longer)
    assert index.publish("ns", "longer", longer) is None
    cache.release("long")
    cache.release("longer")
    cache.check()
    index.clear()
    cache.check()
    assert cache.groups[0].pool.pages_in_use == 0


def test_equal_digests_do_not_confuse_different_prefixes(monkeypatch):
    monkeypatch.setattr(prefix_module, "fnv1a_step", lambda digest, token: 42)
    cache = manager()
    index = PrefixIndex(cache, maximum_entries=8)
    first, second = list(range(10, 19)), list(range(50, 59))
    for name, prompt in (("a", first), ("b", second)):
        run_prompt(cache, name, prompt)
        assert index.publish("ns", name, prompt) is not None
    assert len(index) == 2
    hit_first, hit_second = index.lookup("ns", first), index.lookup("ns", second)
    assert hit_first.tokens == hit_second.tokens == 8 and hit_first.anchor != hit_second.anchor
    assert index.lookup("ns", list(range(90, 99))) is None


def test_with_per_request_state_a_prefix_is_shared_with_the_state_at_its_end():
    """What a model keeps per request beside its pages belongs to a kept prefix as it stood
    at the prefix's end: the request's record is given a copy at that length, the anchor
    takes it over, and a request that adopts the whole prefix starts from it.  Without a
    copy at exactly that length nothing is kept."""
    cache = manager(states={5: StateNeed((3,), torch.float32)})
    index = PrefixIndex(cache, maximum_entries=4)
    prompt = list(range(30, 41))                         # 11 tokens: the prefix is 8
    cache.admit("a")
    cache.extend("a", 8)
    cache.commit("a", 8)
    cache.state(5)[cache.slot("a")] = torch.tensor([1.0, 2.0, 3.0])      # the state after 8
    cache.keep_state("a", 8, cache.snapshot_state("a"))
    cache.extend("a", 11)
    cache.commit("a", 11)
    cache.state(5)[cache.slot("a")] = torch.tensor([9.0, 9.0, 9.0])      # it has moved on
    assert index.publish("ns", "a", prompt) is not None
    cache.release("a")

    match = index.lookup("ns", prompt[:8] + [1, 2])
    assert match is not None and match.tokens == 8
    assert index.lookup("ns", prompt[:4] + [1, 2]) is None               # whole or not at all
    cache.adopt("b", match.anchor, match.tokens)
    assert cache.state(5)[cache.slot("b")].tolist() == [1.0, 2.0, 3.0]
    assert cache.length("b") == 8
    # b goes on and publishes its own, longer prompt: it needs a copy at ITS boundary
    longer = prompt[:8] + list(range(60, 70))            # 18 tokens: the prefix is 16
    cache.extend("b", 18)
    cache.commit("b", 18)
    assert index.publish("ns", "b", longer) is None and index.stats["not_kept"] == 1
    cache.release("b")
    cache.check()
    # a fresh request: the slot is cleared, nothing of b's state is left in it
    cache.admit("c")
    assert cache.state(5)[cache.slot("c")].tolist() == [0.0, 0.0, 0.0]
    cache.release("c")
    index.clear()
    cache.check()
    assert all(group.pool.pages_in_use == 0 for group in cache.groups)


def test_with_a_window_a_prefix_is_shared_whole_or_not_at_all():
    """A windowed group keeps, for a kept prefix, only the pages its window reaches from the
    prefix's end.  A later prompt that goes on from the whole prefix adopts them (the full
    group shares every page, the windowed one the last few); one that departs earlier finds
    nothing; and the pages come back when request and entry have both gone."""
    cache = manager(window=6, slack=1)
    index = PrefixIndex(cache, maximum_entries=4)
    full, windowed = cache.groups
    prompt = list(range(100, 122))                       # 22 tokens: 5 whole pages kept
    cache.admit("a")
    for length in (7, 15, 22):                           # portions: the window passes pages
        cache.extend("a", length)
        cache.commit("a", length)
    assert index.publish("ns", "a", prompt) is not None and index.stats["not_kept"] == 0
    # the request at 20 tokens reads keys 15..19: pages 3 and 4 of the windowed group
    assert cache.anchor_pages() == 5 + 2
    pages_of_a = list(full.host_tables[cache.slot("a")][:5])
    cache.release("a")
    cache.check()
    assert full.pool.pages_in_use == 5 and windowed.pool.pages_in_use == 2

    follow_up = prompt[:20] + [7, 8, 9]
    match = index.lookup("ns", follow_up)
    assert match is not None and match.tokens == 20
    assert index.lookup("ns", prompt[:13] + [1, 2, 3]) is None      # shares three pages only
    assert index.lookup("ns", prompt[:20]) is None                  # one token must still run
    run_prompt(cache, "b", follow_up, adopt=match)
    cache.check()
    table = list(windowed.host_tables[cache.slot("b")][:6])
    assert table[:3] == [-1, -1, -1] and all(page >= 0 for page in table[3:6])
    assert list(full.host_tables[cache.slot("b")][:5]) == pages_of_a
    with pytest.raises(ValueError, match="all of an anchor or none"):
        cache.adopt("c", match.anchor, 8)
    # decoding on: the window passes the shared pages, the entry keeps them alive
    for length in range(24, 40):
        cache.extend("b", length)
        cache.commit("b", length)
        cache.check()
    assert windowed.pool.pages_in_use <= 2 + 4
    cache.release("b")
    index.clear()
    cache.check()
    assert all(group.pool.pages_in_use == 0 for group in cache.groups)


def test_a_prefix_whose_window_pages_are_gone_is_not_kept():
    """Without the page of slack a windowed group may have given back a page that the end of
    the aligned prefix still reads; then nothing is kept and nothing is lost."""
    cache = manager(window=6, slack=0)
    index = PrefixIndex(cache, maximum_entries=4)
    prompt = list(range(50, 73))                         # 23 tokens; aligned prefix 20
    run_prompt(cache, "a", prompt)                       # at 23 the window starts at key 18
    assert index.publish("ns", "a", prompt) is None      # the prefix's end reads key 15
    assert index.stats["not_kept"] == 1 and len(index) == 0 and cache.anchor_pages() == 0
    cache.release("a")
    cache.check()
    assert all(group.pool.pages_in_use == 0 for group in cache.groups)


@pytest.mark.parametrize("seed", range(4))
def test_random_traffic_with_a_window_never_loses_a_page(seed):
    rng = np.random.default_rng(seed)
    cache = manager(num_pages=48, max_requests=4, window=int(rng.integers(3, 14)), slack=1)
    index = PrefixIndex(cache, maximum_entries=4, maximum_page_references=24)
    stem = list(rng.integers(0, 50, size=40))
    live, kept = {}, 0
    for step in range(300):
        action = rng.integers(0, 4)
        if action <= 1 and len(live) < 4:
            # prompts that go on from an aligned cut of the stem: what an earlier one left
            # behind is a whole prefix of a later, longer one
            cut = int(rng.integers(1, 10)) * PAGE
            prompt = stem[:cut] + list(rng.integers(50, 60, size=int(rng.integers(1, 6))))
            name = f"r{step}"
            match = index.lookup("ns", prompt)
            if min(group.pool.free_pages for group in cache.groups) < -(-len(prompt) // PAGE):
                continue
            if match is None:
                cache.admit(name)
            else:
                cache.adopt(name, match.anchor, match.tokens)
                assert tuple(prompt[:match.tokens]) == index._entries[match.anchor].tokens
                kept += 1
            at = cache.length(name)
            while at < len(prompt):                      # portions of changing size
                at = min(len(prompt), at + int(rng.integers(1, 9)))
                cache.extend(name, at)
                cache.commit(name, at)
            live[name] = prompt
            index.publish("ns", name, prompt)
        elif action == 2 and live:
            name = list(live)[int(rng.integers(0, len(live)))]
            cache.release(name)
            del live[name]
        elif action == 3:
            index.evict_for_pressure()
        cache.check()
    assert kept > 0 and index.stats["not_kept"] == 0
    for name in live:
        cache.release(name)
    index.clear()
    cache.check()
    assert all(group.pool.pages_in_use == 0 for group in cache.groups)


def test_random_traffic_never_loses_or_double_frees_a_page():
    rng = np.random.default_rng(0)
    cache = manager(num_pages=40, max_requests=4)
    index = PrefixIndex(cache, maximum_entries=5, maximum_page_references=16)
    stems = [list(rng.integers(0, 50, size=int(n))) for n in (8, 12, 20)]
    live = {}
    for step in range(400):
        action = rng.integers(0, 4)
        if action <= 1 and len(live) < 4:
            stem = stems[int(rng.integers(0, len(stems)))]
            prompt = stem[:int(rng.integers(1, len(stem) + 1))] + \
                list(rng.integers(50, 60, size=int(rng.integers(1, 9))))
            name = f"r{step}"
            match = index.lookup("ns", prompt)
            pages_needed = -(-len(prompt) // PAGE) - (match.tokens // PAGE if match else 0)
            while cache.groups[0].pool.free_pages < pages_needed and index.evict_for_pressure():
                match = index.lookup("ns", prompt)
                pages_needed = -(-len(prompt) // PAGE) - (match.tokens // PAGE if match else 0)
            if cache.groups[0].pool.free_pages < pages_needed:
                continue
            run_prompt(cache, name, prompt, adopt=match)
            if match is not None:
                kept = index._entries[match.anchor].tokens[:match.tokens]
                assert tuple(prompt[:match.tokens]) == kept
            live[name] = prompt
            index.publish("ns", name, prompt)
        elif action == 2 and live:
            name = list(live)[int(rng.integers(0, len(live)))]
            cache.release(name)
            del live[name]
        elif action == 3:
            index.evict_for_pressure()
        cache.check()
        assert index.page_references <= 16 and len(index) <= 5
        assert index.page_references * len(cache.groups) == cache.anchor_pages()
    for name in live:
        cache.release(name)
    index.clear()
    cache.check()
    assert all(group.pool.pages_in_use == 0 for group in cache.groups)


# ------------------------------------------------------------------ with the scheduler

class Rig:
    """Scheduler + cache manager + prefix index on the CPU, wired as the engine wires them,
    with a fake step that 'generates' token 7."""

    def __init__(self, num_pages=16, max_tokens=64, max_running=3, entries=4, index_pages=None):
        self.cache = CacheManager({0: KvNeed(1, 4)}, {}, PAGE, num_pages, max_running, 256,
                                  torch.float32, CPU)
        self.scheduler = FifoScheduler(SchedulerConfig(max_tokens, max_running, None), PAGE)
        self.index = PrefixIndex(self.cache, entries, index_pages)
        self.matches = {}
        self.ran = []          # (request, offset, count) of every portion

    def reusable(self, request):
        match = self.index.lookup(request.namespace, request.feed)
        if match is None:
            return 0
        self.matches[request.id] = match
        return match.tokens

    def admit(self, request_id):
        match = self.matches.pop(request_id, None)
        if match is None:
            self.cache.admit(request_id)
        else:
            self.cache.adopt(request_id, match.anchor, match.tokens)

    def reclaim(self):
        self.matches.clear()
        return self.index.evict_for_pressure()

    def step(self):
        batch = self.scheduler.schedule_iteration(self.cache, self.admit, self.cache.release,
                                                  reusable=self.reusable, reclaim=self.reclaim)
        if batch is None:
            return None
        completions = []
        for work in batch.work:
            request = self.scheduler.request(work.request_id)
            assert self.cache.length(work.request_id) == work.token_offset
            end = work.token_offset + work.token_count
            self.cache.extend(work.request_id, end)
            self.cache.commit(work.request_id, end)
            self.ran.append((work.request_id, work.token_offset, work.token_count))
            if work.kind is WorkKind.PREFILL and work.token_offset < len(request.prompt) <= end:
                self.index.publish(request.namespace, request.id, request.prompt)
            completions.append(WorkCompletion(work.request_id, True,
                                              token=7 if work.samples else None))
        for request in self.scheduler.complete_iteration(batch.id, completions, 256):
            self.cache.release(request.id)
        self.cache.check()
        return batch

    def drain(self):
        steps = 0
        while self.scheduler.has_unfinished():
            assert self.step() is not None, "the scheduler stalled"
            steps += 1
            assert steps < 200


def test_a_reused_prefix_counts_as_progress_at_admission():
    rig = Rig()
    stem = list(range(30, 42))                            # 3 pages
    first = rig.scheduler.submit(stem + [1, 2], 2, namespace="ns")
    rig.drain()
    assert rig.ran[0] == (first, 0, 14)
    second = rig.scheduler.submit(stem + [5, 6, 7], 2, namespace="ns")
    third = rig.scheduler.submit(stem + [9], 2, namespace=None)       # keeps out of the index
    rig.ran.clear()
    rig.drain()
    assert (second, 12, 3) in rig.ran and (third, 0, 13) in rig.ran
    assert rig.scheduler.request(second).reused_tokens == 12
    assert rig.scheduler.request(third).reused_tokens == 0
    assert rig.index.stats["hits"] == 1 and rig.index.stats["reused_tokens"] == 12
    assert len(rig.scheduler.request(second).generated) == 2


def test_kept_prefixes_are_dropped_before_anybody_waits_or_is_preempted():
    # 8 pages; two kept prefixes hold 3 + 3 of them
    rig = Rig(num_pages=8, index_pages=8)
    for base in (100, 200):
        rig.scheduler.submit([base + i for i in range(13)], 1, namespace="ns")
        rig.drain()
    assert len(rig.index) == 2 and rig.cache.groups[0].pool.free_pages == 2
    # a prompt of 5 pages shares nothing.  It first takes the two free pages (a portion of 8
    # tokens); then nobody can move, and the colder prefix goes: its 3 pages are enough.
    big = rig.scheduler.submit(list(range(300, 320)), 1, namespace="ns")
    rig.ran.clear()
    rig.drain()
    assert rig.ran == [(big, 0, 8), (big, 8, 12)]
    assert rig.index.stats["evicted_under_pressure"] == 1
    assert rig.scheduler.stats["preemptions"] == 0
    assert rig.index.lookup("ns", [100 + i for i in range(13)]) is None        # the colder one
    assert rig.index.lookup("ns", [200 + i for i in range(13)]).tokens == 12
    # a prompt that needs every page: the other prefix goes too, before anybody is preempted
    huge = rig.scheduler.submit(list(range(400, 430)), 1, namespace="ns")
    rig.drain()
    assert rig.scheduler.request(huge).generated == [7]
    assert rig.scheduler.stats["preemptions"] == 0
    assert rig.index.stats["evicted_under_pressure"] >= 2
