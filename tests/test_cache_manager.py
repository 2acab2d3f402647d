"""The cache manager on the CPU: no page lost, held twice or freed twice, under random orders
of requests; windows give pages back; reserve/commit/rollback; state slots; sharing."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helix_runtime_b200.cache import CacheManager, KvNeed, OutOfPages, PagePool, StateNeed

CPU = torch.device("cpu")


def manager(num_pages=12, page_size=4, max_requests=4, max_positions=64, window=None,
            states=None, poison=False):
    needs = {0: KvNeed(2, 8), 1: KvNeed(2, 8)}
    if window is not None:
        needs[2] = KvNeed(2, 8, window=window)
        needs[3] = KvNeed(2, 8, window=window)
    return CacheManager(needs, states or {}, page_size, num_pages, max_requests, max_positions,
                        torch.float32, CPU, poison=poison)


def test_pool_is_a_fifo_ring_with_reference_counts():
    pool = PagePool(4)
    assert pool.allocate(3) == [0, 1, 2]
    assert pool.release([1]) == 1
    assert pool.allocate(2) == [3, 1]            # freed pages queue behind the untouched ones
    assert pool.reuse_count == 1
    with pytest.raises(OutOfPages):
        pool.allocate(1)
    pool.share([0])
    assert pool.release([0]) == 0 and pool.release([0]) == 1
    with pytest.raises(RuntimeError, match="more often"):
        pool.release([0])
    with pytest.raises(RuntimeError, match="free"):
        pool.share([0])
    pool.check()


def test_layers_with_the_same_needs_share_a_group_and_windows_get_their_own():
    cache = manager(window=6)
    assert len(cache.groups) == 2
    full, windowed = cache.groups
    assert full.entries == [0, 1] and windowed.entries == [2, 3]
    assert full.storage.shape == (2, 2, 12, 2, 4, 8)
    keys, values = cache.layer_storage(3)
    assert keys.data_ptr() == windowed.storage[1, 0].data_ptr()
    assert cache.bytes_per_token() == 2 * (2 * 2 * 2 * 8 * 4)


def test_reserve_commit_and_rollback():
    cache = manager()
    cache.admit("a")
    assert cache.pages_to_extend("a", 9) == [3]
    cache.extend("a", 9)
    assert cache.length("a") == 0                # nothing is published before the step succeeds
    cache.commit("a", 9)
    assert cache.length("a") == 9
    cache.extend("a", 17)
    cache.rollback("a")                          # the step failed
    assert cache.length("a") == 9 and cache.groups[0].pool.pages_in_use == 3
    with pytest.raises(ValueError, match="never shrinks"):
        cache.extend("a", 4)
    with pytest.raises(ValueError, match="cannot publish"):
        cache.commit("a", 30)
    cache.check()
    assert cache.release("a") == 3
    cache.check()


def test_two_steps_in_flight_reserve_on_top_of_each_other():
    cache = manager()
    cache.admit("a")
    cache.extend("a", 4)
    cache.commit("a", 4)
    cache.extend("a", 5)                         # a step in flight
    cache.extend("a", 9)                         # the step queued behind it
    assert cache.reserved("a") == 9 and cache.length("a") == 4
    assert cache.max_extend("a", 100, [0]) == 3  # counted from what is reserved
    cache.rollback("a", keep_length=5)           # the second failed before it ran
    assert cache.reserved("a") == 5 and cache.groups[0].pool.pages_in_use == 2
    cache.extend("a", 9)
    cache.commit("a", 5)                         # the first succeeded
    assert cache.length("a") == 5 and cache.reserved("a") == 9
    with pytest.raises(ValueError, match="cannot roll back"):
        cache.rollback("a", keep_length=4)
    with pytest.raises(ValueError, match="cannot roll back"):
        cache.rollback("a", keep_length=10)
    cache.rollback("a")                          # the first's successor failed on the device
    assert cache.reserved("a") == 5 and cache.groups[0].pool.pages_in_use == 2
    cache.check()
    cache.release("a")
    cache.check()


def test_running_out_of_pages_takes_nothing():
    cache = manager(num_pages=4)
    cache.admit("a")
    cache.admit("b")
    cache.extend("a", 12)
    with pytest.raises(OutOfPages):
        cache.extend("b", 8)
    assert cache.groups[0].pool.free_pages == 1
    assert cache.max_extend("b", 100) == 4 and cache.max_extend("a", 100) == 4
    assert cache.max_extend_new(100, [0]) == 0
    cache.check()


def test_a_window_gives_pages_back_once_it_has_passed_them():
    cache = manager(num_pages=16, window=6, max_positions=64)
    cache.admit("a")
    windowed = cache.groups[1]
    length = 0
    for step in (5, 4, 1, 1, 1, 8, 1, 1, 1, 1, 20):
        length += step
        cache.extend("a", length)
        cache.commit("a", length)
        cache.check()
        first_needed = max(0, length - 6 + 1)            # oldest key the next query reads
        table = list(windowed.host_tables[cache.slot("a")])
        for index in range(-(-length // 4)):
            if (index + 1) * 4 <= first_needed:
                assert table[index] == -1, f"length {length}: page {index} should be gone"
            else:
                assert table[index] >= 0, f"length {length}: page {index} is still needed"
        assert windowed.pool.pages_in_use <= 3 + -(-step // 4)
    assert cache.groups[0].pool.pages_in_use == -(-length // 4)   # the full group keeps all
    cache.release("a")
    cache.check()
    assert all(group.pool.free_pages == 16 for group in cache.groups)


def test_state_slots_are_zeroed_at_admission_and_reused():
    cache = manager(states={0: StateNeed((3, 2)), 1: StateNeed((5,), torch.int32)})
    slot = cache.admit("a")
    cache.state(0)[slot] += 7.0
    cache.state(1)[slot] += 3
    cache.release("a")
    for name in ("b", "c", "d", "e"):
        cache.admit(name)
    with pytest.raises(OutOfPages, match="slot"):
        cache.admit("f")
    assert float(cache.state(0).abs().sum()) == 0.0 and int(cache.state(1).abs().sum()) == 0
    cache.check()


def test_sharing_a_prefix_of_whole_pages():
    cache = manager()
    cache.admit("a")
    cache.extend("a", 10)
    cache.commit("a", 10)
    with pytest.raises(ValueError, match="multiple of the page size"):
        cache.fork("a", "b", 6)
    with pytest.raises(ValueError, match="published"):
        cache.fork("a", "b", 12)
    cache.fork("a", "b", 8)
    assert cache.length("b") == 8
    pool = cache.groups[0].pool
    shared = list(cache.groups[0].host_tables[cache.slot("b")][:2])
    assert [pool.refcount(page) for page in shared] == [2, 2]
    cache.extend("b", 11)
    cache.commit("b", 11)
    cache.check()
    cache.release("a")                            # shared pages stay with b
    assert [pool.refcount(page) for page in shared] == [1, 1]
    cache.check()
    cache.release("b")
    assert pool.free_pages == pool.num_pages
    cache.check()


def test_poisoned_pages_are_nan_when_free():
    cache = manager(poison=True, num_pages=3)
    assert torch.isnan(cache.groups[0].storage).all()
    cache.admit("a")
    cache.extend("a", 4)
    cache.commit("a", 4)
    page = int(cache.groups[0].host_tables[cache.slot("a")][0])
    cache.groups[0].storage[:, :, page] = 1.0
    cache.release("a")
    assert torch.isnan(cache.groups[0].storage[:, :, page]).all()


def test_groups_with_a_window_may_have_a_pool_of_their_own_size():
    """Two full-attention layers with 12 pages and two windowed layers with 4: a request of 40
    positions holds ten pages of the one and never more than three of the other."""
    needs = {0: KvNeed(2, 8), 1: KvNeed(2, 8), 2: KvNeed(2, 8, window=6), 3: KvNeed(2, 8, window=6)}
    cache = CacheManager(needs, {}, 4, 12, 2, 64, torch.float32, torch.device("cpu"),
                         window_pages={6: 4})
    full, windowed = cache.groups
    assert (full.pool.num_pages, windowed.pool.num_pages) == (12, 4)
    assert full.storage.shape[2] == 12 and windowed.storage.shape[2] == 4
    assert cache.free_pages() == [12, 4]
    cache.admit("a")
    # the small pool limits the portion: 16 tokens of pages at most at once
    assert cache.max_extend("a", 40) == 16
    length = 0
    while length < 40:
        length += cache.max_extend("a", min(5, 40 - length))
        cache.extend("a", length)
        cache.commit("a", length)
        cache.check()
        assert windowed.pool.pages_in_use <= 3
    assert full.pool.pages_in_use == 10
    cache.release("a")
    cache.check()
    with pytest.raises(ValueError, match="no layer has"):
        CacheManager(needs, {}, 4, 12, 2, 64, torch.float32, torch.device("cpu"),
                     window_pages={7: 4})


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests_never_lose_a_page(seed):
    rng = np.random.default_rng(seed)
    window = [None, 5, 9][seed % 3]
    cache = manager(num_pages=10, page_size=4, max_requests=3, max_positions=40, window=window)
    lengths = {}
    counter = 0
    for _ in range(400):
        action = rng.integers(0, 5)
        if action == 0 and cache.free_slots:
            name = f"r{counter}"
            counter += 1
            cache.admit(name)
            lengths[name] = 0
        elif action in (1, 2) and lengths:
            name = list(lengths)[rng.integers(0, len(lengths))]
            grow = int(rng.integers(1, 9))
            target = min(lengths[name] + grow, 40)
            if target == lengths[name]:
                continue
            possible = cache.max_extend(name, target - lengths[name])
            try:
                cache.extend(name, target)
                assert possible >= target - lengths[name]
            except OutOfPages:
                assert possible < target - lengths[name]
                cache.check()
                continue
            if rng.random() < 0.2:
                cache.rollback(name)              # the step failed
            else:
                cache.commit(name, target)
                lengths[name] = target
        elif action == 3 and lengths:
            name = list(lengths)[rng.integers(0, len(lengths))]
            cache.release(name)
            del lengths[name]
        cache.check()
        for name, length in lengths.items():
            assert cache.length(name) == length
    for name in list(lengths):
        cache.release(name)
    cache.check()
    assert all(group.pool.free_pages == group.pool.num_pages for group in cache.groups)
    assert cache.free_slots == 3
    if counter > 6:
        assert any(group.pool.reuse_count > 0 for group in cache.groups)


def test_what_ends_while_a_step_is_queued_is_parked_until_that_step_completes():
    """Pages and the slot of a request that ends while step 7 is on the device stay out of the
    ring until ``settle(7)``; then they return in the order they were parked, so page reuse
    stays a function of the trace.  The reference tests its deferred allocator the same way,
    with completions that the test controls (tests/deferred_allocator_test.cpp:51-160)."""
    cache = CacheManager({0: KvNeed(1, 4)}, {}, 4, 8, 2, 64, torch.float32, torch.device("cpu"))
    cache.admit("a")
    cache.extend("a", 10)
    cache.commit("a", 10)                         # pages 0, 1, 2
    cache.admit("b")
    cache.extend("b", 5)
    cache.commit("b", 5)                          # pages 3, 4
    assert cache.free_pages() == [3] and cache.free_slots == 0
    assert cache.release("a", after=7) == 0       # nothing free yet
    assert cache.free_pages() == [3] and cache.free_slots == 0 and cache.parked_pages == 3
    assert not cache.has("a")
    cache.check()
    with pytest.raises(OutOfPages):               # the slot is parked too
        cache.admit("c")
    assert cache.settle(6) == 0                   # an earlier step completing changes nothing
    cache.extend("b", 9)
    cache.rollback("b", after=7)                  # a failed step's page, also behind step 7
    assert cache.parked_pages == 4 and cache.free_pages() == [2]
    cache.check()
    assert cache.settle(7) == 4
    assert cache.free_pages() == [6] and cache.free_slots == 1 and cache.parked_pages == 0
    cache.admit("c")
    cache.extend("c", 24)
    # the ring: never-used pages 6, 7 first, then a's pages in their order, then b's rolled back
    assert cache._requests["c"].tables[0] == [6, 7, 0, 1, 2, 5]
    # a step that has completed already parks nothing
    assert cache.release("b", after=7) == 2
    cache.release("c")
    cache.check()
    assert cache.free_pages() == [8] and cache.free_slots == 2


def test_random_orders_with_parking_lose_nothing():
    rng = np.random.default_rng(11)
    cache = CacheManager({0: KvNeed(2, 8), 1: KvNeed(2, 8, window=12)}, {}, 4, 24, 4, 96,
                         torch.float32, torch.device("cpu"))
    live, step, settled = {}, 0, -1
    for _ in range(600):
        action = rng.integers(0, 5)
        name = f"r{rng.integers(0, 8)}"
        if action == 0 and name not in live and cache.free_slots:
            cache.admit(name)
            live[name] = 0
        elif action == 1 and name in live:
            grow = int(rng.integers(1, 9))
            target = min(live[name] + grow, 96)
            try:
                cache.extend(name, target)
            except OutOfPages:
                continue
            if rng.integers(0, 4) == 0:
                cache.rollback(name, after=step if rng.integers(0, 2) else None)
            else:
                cache.commit(name, target)
                live[name] = target
        elif action == 2 and name in live:
            cache.release(name, after=step if rng.integers(0, 2) else None)
            del live[name]
        elif action == 3:
            step += 1
        elif action == 4 and settled < step:
            settled = int(rng.integers(settled + 1, step + 1))
            cache.settle(settled)
        cache.check()
    cache.settle(step)
    for name in list(live):
        cache.release(name)
    cache.check()
    assert cache.parked_pages == 0 and cache.free_slots == 4
    assert cache.free_pages() == [24, 24]
