"""Request metrics at an observation time: counts by state, token totals, rates, and the
distributions of waiting time, time to the first token, request latency and the time
between tokens.

The definitions are the reference's (src/scheduler/metrics.cpp:60-150,
include/helix/scheduler/metrics.hpp:11-50): P50 and P95 interpolate linearly between the
sorted samples at ``p * (N - 1)``; latency counts finished requests only (cancelled and
failed ones keep their own counts); waiting time runs from creation to the first time the
request was given work, time to the first token from creation to the first sampled token;
rates are defined only for a positive window that begins at the earliest creation time.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Iterable, List

from .scheduler import Request, RequestState


@dataclasses.dataclass(frozen=True)
class DurationStatistics:
    sample_count: int = 0
    minimum_seconds: float = 0.0
    mean_seconds: float = 0.0
    p50_seconds: float = 0.0
    p95_seconds: float = 0.0
    maximum_seconds: float = 0.0


@dataclasses.dataclass(frozen=True)
class SchedulerMetrics:
    request_count: int = 0
    waiting_count: int = 0
    prefill_count: int = 0
    decoding_count: int = 0
    finished_count: int = 0
    cancelled_count: int = 0
    failed_count: int = 0
    prompt_tokens_processed: int = 0
    generated_tokens: int = 0
    observation_seconds: float = 0.0
    throughput_defined: bool = False
    finished_requests_per_second: float = 0.0
    generated_tokens_per_second: float = 0.0
    processed_tokens_per_second: float = 0.0
    waiting_time: DurationStatistics = DurationStatistics()
    time_to_first_token: DurationStatistics = DurationStatistics()
    request_latency: DurationStatistics = DurationStatistics()
    inter_token_latency: DurationStatistics = DurationStatistics()


def interpolated_percentile(sorted_samples: List[float], probability: float) -> float:
    if not sorted_samples:
        raise ValueError("a percentile needs at least one sample")
    position = probability * (len(sorted_samples) - 1)
    lower, upper = math.floor(position), math.ceil(position)
    fraction = position - lower
    return sorted_samples[lower] + (sorted_samples[upper] - sorted_samples[lower]) * fraction


def summarize_durations(samples: Iterable[float]) -> DurationStatistics:
    ordered = sorted(samples)
    if not ordered:
        return DurationStatistics()
    return DurationStatistics(
        sample_count=len(ordered), minimum_seconds=ordered[0],
        mean_seconds=sum(ordered) / len(ordered),
        p50_seconds=interpolated_percentile(ordered, 0.50),
        p95_seconds=interpolated_percentile(ordered, 0.95), maximum_seconds=ordered[-1])


_COUNTER = {RequestState.WAITING: "waiting_count", RequestState.PREFILL: "prefill_count",
            RequestState.DECODING: "decoding_count", RequestState.FINISHED: "finished_count",
            RequestState.CANCELLED: "cancelled_count", RequestState.FAILED: "failed_count"}


def summarize_request_metrics(requests: Iterable[Request], observed_at: float) -> SchedulerMetrics:
    requests = list(requests)
    if not requests:
        return SchedulerMetrics()
    counts = {name: 0 for name in _COUNTER.values()}
    seen = set()
    waiting, first_token, latency, between = [], [], [], []
    prompt_tokens = generated_tokens = 0
    earliest = observed_at
    for request in requests:
        if request.id in seen:
            raise ValueError(f"request {request.id} appears twice")
        seen.add(request.id)
        if observed_at < request.latest_event_at:
            raise ValueError(f"the observation time precedes what request {request.id} has done")
        earliest = min(earliest, request.created_at)
        counts[_COUNTER[request.state]] += 1
        prompt_tokens += request.prompt_tokens_processed
        generated_tokens += len(request.generated)
        if request.first_scheduled_at is not None:
            waiting.append(request.first_scheduled_at - request.created_at)
        if request.first_token_at is not None:
            first_token.append(request.first_token_at - request.created_at)
        if request.state is RequestState.FINISHED:
            latency.append(request.finished_at - request.created_at)
        times = request.token_times
        between.extend(later - earlier for earlier, later in zip(times, times[1:]))
    window = observed_at - earliest
    defined = window > 0.0
    return SchedulerMetrics(
        request_count=len(requests), prompt_tokens_processed=prompt_tokens,
        generated_tokens=generated_tokens, observation_seconds=window, throughput_defined=defined,
        finished_requests_per_second=counts["finished_count"] / window if defined else 0.0,
        generated_tokens_per_second=generated_tokens / window if defined else 0.0,
        processed_tokens_per_second=(prompt_tokens + generated_tokens) / window if defined else 0.0,
        waiting_time=summarize_durations(waiting),
        time_to_first_token=summarize_durations(first_token),
        request_latency=summarize_durations(latency),
        inter_token_latency=summarize_durations(between), **counts)
