"""The scheduler's decisions, driven with fake completions on the CPU (as the reference tests
its scheduler, tests/fifo_scheduler_test.cpp): batch membership, portions under the token
budget, decoding, finishing and freeing, and what happens when pages run out."""
from __future__ import annotations

import pytest
import torch

from helix_runtime_b200.cache import CacheManager, KvNeed
from helix_runtime_b200.engine import (FifoScheduler, RequestState, SchedulerConfig, StopReason,
                                       WorkCompletion, WorkKind)


class Rig:
    """Scheduler + a real cache manager on the CPU + a fake step that 'generates' token 7."""

    def __init__(self, num_pages=16, page_size=4, max_tokens=8, max_running=3, chunk=None,
                 max_positions=64, token=7):
        self.cache = CacheManager({0: KvNeed(1, 4)}, {}, page_size, num_pages, max_running,
                                  max_positions, torch.float32, torch.device("cpu"))
        self.scheduler = FifoScheduler(SchedulerConfig(max_tokens, max_running, chunk), page_size)
        self.max_positions = max_positions
        self.token = token
        self.appended = 0

    def step(self, fail=()):
        batch = self.scheduler.schedule_iteration(self.cache, self.cache.admit, self.cache.release)
        if batch is None:
            return None, []
        completions = []
        for work in batch.work:
            request = self.scheduler.request(work.request_id)
            assert self.cache.length(work.request_id) == work.token_offset
            if work.request_id in fail:
                completions.append(WorkCompletion(work.request_id, False, error="injected"))
                continue
            self.cache.extend(work.request_id, work.token_offset + work.token_count)
            self.cache.commit(work.request_id, work.token_offset + work.token_count)
            self.appended += work.token_count
            token = self.token(request) if callable(self.token) else self.token
            completions.append(WorkCompletion(work.request_id, True,
                                              token=token if work.samples else None))
        retired = self.scheduler.complete_iteration(batch.id, completions, self.max_positions)
        for request in retired:
            if self.cache.has(request.id):
                self.cache.release(request.id)
        self.cache.check()
        return batch, retired

    def drain(self, limit=200):
        steps = 0
        while self.scheduler.has_unfinished():
            batch, _ = self.step()
            assert batch is not None, "the scheduler stalled"
            steps += 1
            assert steps < limit
        return steps


def summary(batch):
    return [(w.request_id, w.kind, w.token_offset, w.token_count, w.samples) for w in batch.work]


def test_prompt_is_cut_under_the_token_budget_and_rows_written_are_p_plus_n_minus_1():
    # the reference's own example: P=3, N=3, budget 2 -> 5 cache rows
    # (tests/cpu_runtime_engine_test.cpp:137, 143)
    rig = Rig(max_tokens=2)
    rid = rig.scheduler.submit([1, 2, 3], max_new_tokens=3)
    batch, _ = rig.step()
    assert summary(batch) == [(rid, WorkKind.PREFILL, 0, 2, False)]
    batch, _ = rig.step()
    assert summary(batch) == [(rid, WorkKind.PREFILL, 2, 1, True)]
    assert rig.scheduler.request(rid).state is RequestState.DECODING
    batch, _ = rig.step()
    assert summary(batch) == [(rid, WorkKind.DECODE, 3, 1, True)]
    batch, retired = rig.step()
    assert [r.id for r in retired] == [rid]
    request = rig.scheduler.request(rid)
    assert request.generated == [7, 7, 7] and request.stop_reason is StopReason.MAX_NEW_TOKENS
    assert rig.appended == 3 + 3 - 1
    assert not rig.scheduler.has_unfinished() and rig.cache.free_pages() == [16]


def test_running_requests_come_first_then_the_queue_in_order():
    rig = Rig(max_tokens=8, max_running=2)
    a = rig.scheduler.submit([1] * 5, 4)
    b = rig.scheduler.submit([2] * 6, 4)
    c = rig.scheduler.submit([3] * 2, 4)
    batch, _ = rig.step()
    assert summary(batch) == [(a, WorkKind.PREFILL, 0, 5, True), (b, WorkKind.PREFILL, 0, 3, False)]
    assert batch.budget_exhausted
    batch, _ = rig.step()           # a decodes beside the rest of b's prompt; c waits for a slot
    assert summary(batch) == [(a, WorkKind.DECODE, 5, 1, True), (b, WorkKind.PREFILL, 3, 3, True)]
    assert rig.scheduler.request(c).state is RequestState.WAITING
    rig.drain()
    assert [rig.scheduler.request(r).generated for r in (a, b, c)] == [[7] * 4] * 3


def test_prefill_chunk_knob_mixes_portions_with_decode_tokens():
    rig = Rig(max_tokens=64, max_running=3, chunk=4, num_pages=32)
    a = rig.scheduler.submit([1] * 3, 6)
    rig.step()
    b = rig.scheduler.submit([2] * 10, 2)
    batch, _ = rig.step()
    assert summary(batch) == [(a, WorkKind.DECODE, 3, 1, True), (b, WorkKind.PREFILL, 0, 4, False)]
    batch, _ = rig.step()
    assert summary(batch) == [(a, WorkKind.DECODE, 4, 1, True), (b, WorkKind.PREFILL, 4, 4, False)]
    batch, _ = rig.step()
    assert summary(batch) == [(a, WorkKind.DECODE, 5, 1, True), (b, WorkKind.PREFILL, 8, 2, True)]


def test_a_portion_may_be_made_to_end_at_the_prompts_last_page_boundary():
    """For models that keep state beside their pages: some step ends exactly where the
    prompt's longest page-aligned prefix ends (pages of 4: 8 of 11 tokens), whatever the
    budget and the chunk size would have cut; a prompt that ends on a boundary, or that is
    shorter than a page, is not cut."""
    rig = Rig(max_tokens=64, max_running=3, num_pages=32)
    rig.scheduler = FifoScheduler(SchedulerConfig(64, 3, None, cut_prompt_at_last_page=True), 4)
    a = rig.scheduler.submit([1] * 11, 2)
    b = rig.scheduler.submit([2] * 8, 2)
    c = rig.scheduler.submit([3] * 3, 2)
    batch, _ = rig.step()
    assert summary(batch) == [(a, WorkKind.PREFILL, 0, 8, False), (b, WorkKind.PREFILL, 0, 8, True),
                              (c, WorkKind.PREFILL, 0, 3, True)]
    batch, _ = rig.step()
    assert summary(batch)[0] == (a, WorkKind.PREFILL, 8, 3, True)
    rig.drain()
    # with a chunk of 5 the boundary at 8 is met by cutting the second chunk short
    rig = Rig(max_tokens=64, max_running=3, num_pages=32)
    rig.scheduler = FifoScheduler(SchedulerConfig(64, 3, 5, cut_prompt_at_last_page=True), 4)
    a = rig.scheduler.submit([1] * 11, 2)
    cuts = []
    while rig.scheduler.request(a).state is not RequestState.DECODING:
        batch, _ = rig.step()
        cuts.append(summary(batch)[0][2:4])
    assert cuts == [(0, 5), (5, 3), (8, 3)]


def test_eos_ends_a_request_and_the_token_is_emitted():
    rig = Rig(token=lambda request: 9 if len(request.generated) == 2 else 7)
    rid = rig.scheduler.submit([1, 2], max_new_tokens=10, eos_token=9)
    rig.drain()
    request = rig.scheduler.request(rid)
    assert request.generated == [7, 7, 9] and request.stop_reason is StopReason.EOS_TOKEN


def test_zero_new_tokens_runs_the_prompt_and_finishes():
    rig = Rig()
    rid = rig.scheduler.submit([1, 2, 3], max_new_tokens=0)
    rig.drain()
    request = rig.scheduler.request(rid)
    assert request.generated == [] and request.state is RequestState.FINISHED


def test_context_limit_stops_generation():
    rig = Rig(max_positions=6, num_pages=4, max_tokens=8)
    rid = rig.scheduler.submit([1, 2, 3, 4], max_new_tokens=50)
    rig.drain()
    request = rig.scheduler.request(rid)
    # positions 0..5 hold the prompt and two fed-back tokens; the third token is emitted
    assert len(request.generated) == 3 and request.stop_reason is StopReason.CONTEXT_LIMIT


def test_when_pages_run_out_the_head_waits_and_is_not_skipped():
    rig = Rig(num_pages=3, page_size=4, max_tokens=32, max_running=3)
    a = rig.scheduler.submit([1] * 8, 3)        # 2 pages, then a third while decoding
    b = rig.scheduler.submit([2] * 8, 2)        # cannot start while a holds the pool
    c = rig.scheduler.submit([3] * 2, 2)        # would fit, but must not overtake b
    batch, _ = rig.step()
    assert summary(batch) == [(a, WorkKind.PREFILL, 0, 8, True), (b, WorkKind.PREFILL, 0, 4, False)]
    assert batch.kv_limited
    batch, _ = rig.step()
    # a needs a third page for position 8, b holds it: a gets nothing, planning stops there
    # and the youngest running request (b) is preempted so that a can go on
    assert batch.preempted == [b]
    assert summary(batch) == [(a, WorkKind.DECODE, 8, 1, True)]
    assert rig.scheduler.request(b).state is RequestState.WAITING
    assert rig.scheduler.request(c).state is RequestState.WAITING
    assert list(rig.scheduler.waiting) == [b, c]
    rig.drain()
    for rid, count in ((a, 3), (b, 2), (c, 2)):
        assert rig.scheduler.request(rid).generated == [7] * count
    assert rig.scheduler.stats["preemptions"] >= 1
    assert rig.cache.free_pages() == [3]


def test_a_preempted_request_recomputes_its_prompt_and_what_it_had_generated():
    rig = Rig(num_pages=4, page_size=4, max_tokens=32, max_running=2)
    a = rig.scheduler.submit([1] * 7, 6)
    b = rig.scheduler.submit([2] * 7, 6)
    seen = []
    while rig.scheduler.has_unfinished():
        batch, _ = rig.step()
        seen.append(summary(batch))
        assert len(seen) < 50
    request = rig.scheduler.request(b)
    assert request.preemptions >= 1 and request.generated == [7] * 6
    resumed = [w for step in seen for w in step if w[0] == b and w[1] is WorkKind.PREFILL]
    restart = max(index for index, work in enumerate(resumed) if work[2] == 0)
    assert restart > 0                                      # it started from position 0 again
    assert sum(work[3] for work in resumed[restart:]) > 7   # prompt + its generated tokens


def test_failed_work_fails_the_request_and_frees_its_pages():
    rig = Rig()
    a = rig.scheduler.submit([1] * 5, 4)
    b = rig.scheduler.submit([2] * 3, 4)
    batch, retired = rig.step(fail={a})
    assert [r.id for r in retired] == [a]
    assert rig.scheduler.request(a).state is RequestState.FAILED
    assert rig.scheduler.request(a).error == "injected"
    rig.drain()
    assert rig.scheduler.request(b).generated == [7] * 4 and rig.cache.free_pages() == [16]


def test_cancel_and_bad_submissions():
    rig = Rig()
    a = rig.scheduler.submit([1] * 5, 4)
    rig.step()
    assert rig.scheduler.cancel(a) and not rig.scheduler.cancel(a)
    rig.cache.release(a)
    assert rig.scheduler.request(a).stop_reason is StopReason.CANCELLED
    assert not rig.scheduler.has_unfinished()
    with pytest.raises(ValueError):
        rig.scheduler.submit([], 4)
    with pytest.raises(ValueError):
        rig.scheduler.submit([1], -1)
    with pytest.raises(ValueError):
        rig.scheduler.submit([1], 1, temperature=-0.5)


def test_completions_are_validated_before_anything_changes():
    rig = Rig()
    a = rig.scheduler.submit([1] * 3, 2)
    batch = rig.scheduler.schedule_iteration(rig.cache, rig.cache.admit, rig.cache.release)
    with pytest.raises(RuntimeError, match="in flight"):
        rig.scheduler.schedule_iteration(rig.cache, rig.cache.admit, rig.cache.release)
    with pytest.raises(ValueError, match="one completion per work item"):
        rig.scheduler.complete_iteration(batch.id, [], 64)
    with pytest.raises(ValueError, match="no token"):
        rig.scheduler.complete_iteration(batch.id, [WorkCompletion(a, True)], 64)
    with pytest.raises(RuntimeError, match="no such iteration"):
        rig.scheduler.complete_iteration(batch.id + 1, [WorkCompletion(a, True, token=1)], 64)
    assert rig.scheduler.request(a).processed == 0
    rig.scheduler.complete_iteration(batch.id, [WorkCompletion(a, True, token=1)], 64)
    assert rig.scheduler.request(a).generated == [1]


def test_many_requests_through_a_small_pool_all_finish_and_nothing_leaks():
    rig = Rig(num_pages=8, page_size=4, max_tokens=16, max_running=4, max_positions=32)
    ids = [rig.scheduler.submit([i % 5 + 1] * (1 + (i * 7) % 13), 1 + (i * 3) % 6)
           for i in range(32)]
    rig.drain(limit=2000)
    for i, rid in enumerate(ids):
        request = rig.scheduler.request(rid)
        assert request.state is RequestState.FINISHED
        assert len(request.generated) == 1 + (i * 3) % 6
    assert rig.cache.free_pages() == [8] and rig.cache.free_slots == 4
    assert rig.cache.groups[0].pool.reuse_count > 0


# ----------------------------------------------------------------- planning ahead

class AheadRig(Rig):
    """Drives the scheduler the way the engine does with lookahead: the iteration after the
    one in flight is planned (and its cache rows reserved) before that one is completed."""

    def launch(self, batch):
        for work in batch.work:
            reserved = self.cache.reserved(work.request_id)
            assert reserved == work.token_offset
            self.cache.extend(work.request_id, reserved + work.token_count)

    def complete(self, batch, tokens):
        completions = []
        for work in batch.work:
            request = self.scheduler.request(work.request_id)
            if self.cache.has(work.request_id):
                self.cache.commit(work.request_id, work.token_offset + work.token_count)
            completions.append(WorkCompletion(work.request_id, True,
                                              token=tokens.get(request.id, 7)))
        retired = self.scheduler.complete_iteration(batch.id, completions, self.max_positions)
        for request in retired:
            if self.cache.has(request.id):
                self.cache.release(request.id)
        self.cache.check()
        return retired


def decoding_rig(**options):
    rig = AheadRig(**options)
    ids = [rig.scheduler.submit([1, 2, 3], max_new_tokens=6, eos_token=9) for _ in range(2)]
    rig.step()                                     # both prompts whole; first tokens sampled
    return rig, ids


def test_the_next_decode_iteration_is_planned_before_the_one_in_flight_completes():
    rig, ids = decoding_rig()
    first = rig.scheduler.schedule_iteration(rig.cache, rig.cache.admit, rig.cache.release)
    rig.launch(first)
    ahead = rig.scheduler.schedule_ahead(rig.cache, rig.max_positions)
    assert summary(ahead) == [(ids[0], WorkKind.DECODE, 4, 1, True),
                              (ids[1], WorkKind.DECODE, 4, 1, True)]
    assert ahead.id == first.id + 1
    assert rig.scheduler.schedule_ahead(rig.cache, rig.max_positions) is None   # only one ahead
    rig.launch(ahead)
    assert rig.complete(first, {}) == []
    assert rig.scheduler.active is ahead and rig.scheduler.ahead is None
    with pytest.raises(RuntimeError, match="in flight"):
        rig.scheduler.schedule_iteration(rig.cache, rig.cache.admit, rig.cache.release)
    rig.complete(ahead, {})
    for rid in ids:
        request = rig.scheduler.request(rid)
        assert request.generated == [7, 7, 7] and request.processed == 5
        assert rig.cache.length(rid) == 5


def test_a_request_that_ends_in_flight_loses_its_row_of_the_iteration_planned_ahead():
    rig, ids = decoding_rig()
    first = rig.scheduler.schedule_iteration(rig.cache, rig.cache.admit, rig.cache.release)
    rig.launch(first)
    ahead = rig.scheduler.schedule_ahead(rig.cache, rig.max_positions)
    rig.launch(ahead)
    retired = rig.complete(first, {ids[0]: 9})              # end of sequence for the first
    assert [r.id for r in retired] == [ids[0]]
    assert not rig.cache.has(ids[0])                        # pages back while its row is in flight
    assert rig.complete(ahead, {}) == []
    gone, stays = rig.scheduler.request(ids[0]), rig.scheduler.request(ids[1])
    assert gone.generated == [7, 9] and gone.stop_reason is StopReason.EOS_TOKEN
    assert stays.generated == [7, 7, 7]
    # the next plan ahead holds the remaining request only
    second = rig.scheduler.schedule_iteration(rig.cache, rig.cache.admit, rig.cache.release)
    rig.launch(second)
    assert summary(rig.scheduler.schedule_ahead(rig.cache, rig.max_positions)) == \
        [(ids[1], WorkKind.DECODE, 6, 1, True)]


def test_nothing_is_planned_ahead_when_its_make_up_depends_on_the_tokens_in_flight():
    # a request that reaches its count of new tokens in the iteration in flight
    rig = AheadRig()
    rid = rig.scheduler.submit([1, 2, 3], max_new_tokens=3)
    rig.step()
    batch = rig.scheduler.schedule_iteration(rig.cache, rig.cache.admit, rig.cache.release)
    rig.launch(batch)
    assert rig.scheduler.request(rid).remaining_generation == 2
    assert rig.scheduler.schedule_ahead(rig.cache, rig.max_positions) is not None
    rig.launch(rig.scheduler.ahead)
    rig.complete(batch, {})
    assert rig.scheduler.schedule_ahead(rig.cache, rig.max_positions) is None   # last token next
    assert [r.id for r in rig.complete(rig.scheduler.active, {})] == [rid]

    # a prompt portion in the batch
    rig = AheadRig(max_tokens=2)
    rig.scheduler.submit([1, 2, 3], max_new_tokens=4)
    batch = rig.scheduler.schedule_iteration(rig.cache, rig.cache.admit, rig.cache.release)
    rig.launch(batch)
    assert rig.scheduler.schedule_ahead(rig.cache, rig.max_positions) is None

    # somebody waits who could be admitted
    rig, ids = decoding_rig()
    rig.scheduler.submit([4, 5], max_new_tokens=2)
    batch = rig.scheduler.schedule_iteration(rig.cache, rig.cache.admit, rig.cache.release)
    assert len(batch.work) == 3

    # the context limit ends the request in the iteration in flight
    rig = AheadRig(max_positions=5)
    rig.scheduler.submit([1, 2, 3], max_new_tokens=10)
    rig.step()
    batch = rig.scheduler.schedule_iteration(rig.cache, rig.cache.admit, rig.cache.release)
    rig.launch(batch)                                           # position 3
    assert rig.scheduler.schedule_ahead(rig.cache, rig.max_positions) is not None  # position 4
    rig.launch(rig.scheduler.ahead)
    rig.complete(batch, {})
    assert rig.scheduler.schedule_ahead(rig.cache, rig.max_positions) is None   # no position 5

    # no page for one more token: the ordinary plan decides who waits
    rig = AheadRig(num_pages=2, page_size=4, max_running=2)
    ids = [rig.scheduler.submit([1, 2, 3], max_new_tokens=8) for _ in range(2)]
    rig.step()
    batch = rig.scheduler.schedule_iteration(rig.cache, rig.cache.admit, rig.cache.release)
    rig.launch(batch)                                           # both fill their only page
    assert rig.scheduler.schedule_ahead(rig.cache, rig.max_positions) is None
    rig.complete(batch, {})


def test_a_full_house_plans_ahead_although_others_wait():
    rig = AheadRig(max_running=2)
    ids = [rig.scheduler.submit([1, 2, 3], max_new_tokens=6) for _ in range(3)]
    rig.step()                                                  # two run, the third waits
    batch = rig.scheduler.schedule_iteration(rig.cache, rig.cache.admit, rig.cache.release)
    assert [w.request_id for w in batch.work] == ids[:2]
    rig.launch(batch)
    assert rig.scheduler.schedule_ahead(rig.cache, rig.max_positions) is not None
