"""Request metrics: the reference's definitions (src/scheduler/metrics.cpp,
tests/scheduler_metrics_test.cpp): interpolated percentiles, latency of finished requests
only, rates over the window from the earliest creation."""
from __future__ import annotations

import pytest
import torch

from helix_runtime_b200.cache import CacheManager, KvNeed
from helix_runtime_b200.engine import (DurationStatistics, FifoScheduler, SchedulerConfig,
                                       WorkCompletion, observe)


def test_percentiles_interpolate_between_sorted_samples():
    summary = DurationStatistics.of([8.0, 1.0, 4.0, 2.0])
    assert (summary.sample_count, summary.minimum_seconds, summary.maximum_seconds) == (4, 1.0, 8.0)
    assert summary.mean_seconds == pytest.approx(3.75)
    assert summary.p50_seconds == pytest.approx(3.0)                    # position 1.5
    assert summary.p95_seconds == pytest.approx(4.0 + 0.85 * 4.0)       # position 2.85
    assert DurationStatistics.of([7.0]).p95_seconds == 7.0
    # events that have not happened are NaN and do not count
    assert DurationStatistics.of([float("nan"), 2.0]).sample_count == 1
    assert DurationStatistics.of([]) == DurationStatistics()


def drive(scheduler, cache, now, token=7):
    batch = scheduler.schedule_iteration(cache, cache.admit, cache.release, now=now)
    completions = []
    for work in batch.work:
        cache.extend(work.request_id, work.token_offset + work.token_count)
        cache.commit(work.request_id, work.token_offset + work.token_count)
        completions.append(WorkCompletion(work.request_id, True, token=token if work.samples else None))
    for request in scheduler.complete_iteration(batch.id, completions, 64, now=now + 0.5):
        cache.release(request.id)


def test_metrics_of_a_small_run():
    cache = CacheManager({0: KvNeed(1, 4)}, {}, 4, 16, 2, 64, torch.float32, torch.device("cpu"))
    scheduler = FifoScheduler(SchedulerConfig(8, 2), 4)
    assert observe([], 5.0).request_count == 0
    first = scheduler.submit([1, 2, 3], max_new_tokens=3, now=10.0)
    second = scheduler.submit([4, 5], max_new_tokens=2, now=11.0)
    third = scheduler.submit([6], max_new_tokens=5, now=12.0)        # waits: two run at a time
    drive(scheduler, cache, 20.0)        # both prompts; first tokens at 20.5
    drive(scheduler, cache, 21.0)        # second tokens at 21.5; the second request finishes
    scheduler.cancel(first, now=22.0)
    metrics = observe(scheduler.requests.values(), 30.0)
    assert (metrics.request_count, metrics.waiting_count, metrics.finished_count,
            metrics.cancelled_count, metrics.decoding_count) == (3, 1, 1, 1, 0)
    assert metrics.prompt_tokens_processed == 5 and metrics.generated_tokens == 4
    assert metrics.observation_seconds == pytest.approx(20.0) and metrics.throughput_defined
    assert metrics.generated_tokens_per_second == pytest.approx(4 / 20.0)
    assert metrics.processed_tokens_per_second == pytest.approx(9 / 20.0)
    assert metrics.finished_requests_per_second == pytest.approx(1 / 20.0)
    # waiting: 20 - 10 and 20 - 11; the third has never been given work
    assert metrics.waiting_time.sample_count == 2
    assert metrics.waiting_time.mean_seconds == pytest.approx(9.5)
    assert metrics.time_to_first_token.minimum_seconds == pytest.approx(9.5)      # 20.5 - 11
    assert metrics.time_to_first_token.maximum_seconds == pytest.approx(10.5)
    # latency counts the finished request only: created 11, done 21.5
    assert metrics.request_latency.sample_count == 1
    assert metrics.request_latency.p50_seconds == pytest.approx(10.5)
    assert metrics.inter_token_latency.sample_count == 2
    assert metrics.inter_token_latency.p95_seconds == pytest.approx(1.0)
    assert scheduler.request(third).first_scheduled_at is None
    with pytest.raises(ValueError, match="precedes"):
        observe(scheduler.requests.values(), 21.0)
    with pytest.raises(ValueError, match="twice"):
        observe([scheduler.request(first)] * 2, 30.0)
    # no window, no rates
    alone = FifoScheduler(SchedulerConfig(8, 2), 4)
    alone.submit([1], max_new_tokens=1, now=3.0)
    assert not observe(alone.requests.values(), 3.0).throughput_defined
