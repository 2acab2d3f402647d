"""What the engine's requests have done up to an observation time.

One pass over the requests fills a table (one row per request: state, token counts, the four
time stamps, NaN where an event has not happened); every figure is then a column operation on
that table.  The figures and their definitions are the reference's
(include/helix/scheduler/metrics.hpp:11-50, src/scheduler/metrics.cpp:60-150), so that the
two engines can be compared number by number:

* counts by state; prompt tokens processed and tokens generated;
* rates over the window from the earliest creation time to the observation, defined only
  when that window is positive;
* waiting time (creation to the first time the request was given work), time to the first
  token, latency (finished requests only; cancelled and failed ones are counted, not timed)
  and time between consecutive tokens, each as count / min / mean / P50 / P95 / max, the
  percentiles interpolated linearly between the sorted samples at ``p * (N - 1)``.
"""
from __future__ import annotations

import dataclasses
from typing import Iterable, Sequence

import numpy as np

from .scheduler import Request, RequestState


@dataclasses.dataclass(frozen=True)
class DurationStatistics:
    sample_count: int = 0
    minimum_seconds: float = 0.0
    mean_seconds: float = 0.0
    p50_seconds: float = 0.0
    p95_seconds: float = 0.0
    maximum_seconds: float = 0.0

    @classmethod
    def of(cls, seconds: Sequence[float]) -> "DurationStatistics":
        """Summary of the samples that are there (NaN marks an event that has not happened)."""
        column = np.asarray(seconds, dtype=np.float64).reshape(-1)
        column = column[~np.isnan(column)]
        if column.size == 0:
            return cls()
        p50, p95 = np.percentile(column, (50.0, 95.0), method="linear")
        return cls(int(column.size), float(column.min()), float(column.mean()), float(p50),
                   float(p95), float(column.max()))


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


_STATES = tuple(RequestState)
_NEVER = float("nan")


def observe(requests: Iterable[Request], observed_at: float) -> SchedulerMetrics:
    """The metrics of ``requests`` as seen at ``observed_at`` (the clock of the time stamps)."""
    requests = list(requests)
    if not requests:
        return SchedulerMetrics()
    ids, holders = np.unique([request.id for request in requests], return_counts=True)
    if (holders > 1).any():
        raise ValueError(f"request {int(ids[holders > 1][0])} appears twice")
    # columns: created, first given work, first token, finished
    stamps = np.array([[request.created_at,
                        _NEVER if request.first_scheduled_at is None else request.first_scheduled_at,
                        _NEVER if request.first_token_at is None else request.first_token_at,
                        _NEVER if request.finished_at is None else request.finished_at]
                       for request in requests], dtype=np.float64)
    last_token = np.array([request.token_times[-1] if request.token_times else _NEVER
                           for request in requests], dtype=np.float64)
    latest = np.nanmax(np.column_stack([stamps, last_token]), axis=1)
    early = np.flatnonzero(latest > observed_at)
    if early.size:
        raise ValueError(f"the observation time precedes what request "
                         f"{requests[int(early[0])].id} has done")
    state = np.array([_STATES.index(request.state) for request in requests])
    per_state = np.bincount(state, minlength=len(_STATES))
    counts = {f"{kind.value}_count": int(per_state[index]) for index, kind in enumerate(_STATES)}
    prompt_tokens = int(sum(request.prompt_tokens_processed for request in requests))
    generated = int(sum(len(request.generated) for request in requests))

    created = stamps[:, 0]
    finished = state == _STATES.index(RequestState.FINISHED)
    gaps = [np.diff(np.asarray(request.token_times, dtype=np.float64))
            for request in requests if len(request.token_times) > 1]
    window = float(observed_at - created.min())
    per_second = (lambda amount: amount / window) if window > 0.0 else (lambda amount: 0.0)
    return SchedulerMetrics(
        request_count=len(requests), prompt_tokens_processed=prompt_tokens,
        generated_tokens=generated, observation_seconds=window, throughput_defined=window > 0.0,
        finished_requests_per_second=per_second(counts["finished_count"]),
        generated_tokens_per_second=per_second(generated),
        processed_tokens_per_second=per_second(prompt_tokens + generated),
        waiting_time=DurationStatistics.of(stamps[:, 1] - created),
        time_to_first_token=DurationStatistics.of(stamps[:, 2] - created),
        request_latency=DurationStatistics.of((stamps[:, 3] - created)[finished]),
        inter_token_latency=DurationStatistics.of(np.concatenate(gaps) if gaps else ()),
        **counts)
