"""What the C and C++ interface of the engine (``include/helix_b200/engine.h``) calls.

The interface library hosts this package in an embedded interpreter and keeps one
:class:`~helix_runtime_b200.engine.engine.Engine` per handle, so a C++ program drives the
same scheduler, cache manager, step function and kernels as a Python program: there is one
engine, with two faces.  Every function here takes and returns plain values (integers, floats,
strings, tuples, lists), which is all the C side has to convert.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

from .engine.engine import Engine
from .engine.scheduler import RequestState

STATES = tuple(state.value for state in RequestState)


def create(model_path: str, dtype: str, device: int, page_size: int, num_pages: int,
           max_running_requests: int, max_tokens_per_iteration: int, max_prefill_chunk: int,
           prefix_cache_entries: int, cuda_graphs: int, lookahead: int) -> Engine:
    """An engine over the model at ``model_path`` (a folder or a Helix model file).  Zero for
    ``num_pages`` and ``max_prefill_chunk`` means the engine's default."""
    options = dict(page_size=page_size, max_running_requests=max_running_requests,
                   max_tokens_per_iteration=max_tokens_per_iteration,
                   prefix_cache_entries=prefix_cache_entries, cuda_graphs=bool(cuda_graphs),
                   lookahead=bool(lookahead))
    if num_pages > 0:
        options["num_pages"] = num_pages
    if max_prefill_chunk > 0:
        options["max_prefill_chunk"] = max_prefill_chunk
    return Engine.from_pretrained(model_path, dtype=dtype, device=f"cuda:{device}", **options)


def submit(engine: Engine, tokens: List[int], max_new_tokens: int, eos_token: int,
           temperature: float, seed: int) -> int:
    return engine.submit(tokens, max_new_tokens, None if eos_token < 0 else eos_token,
                         temperature, seed)


def run_iteration(engine: Engine) -> Tuple[int, int, int, int, int, int, int, int]:
    result = engine.run_iteration()
    return (int(result.idle), result.scheduled_tokens, result.prefill_tokens,
            result.decode_tokens, result.sampled, len(result.retired), len(result.preempted),
            int(result.kv_limited))


def run_until_done(engine: Engine, max_iterations: int) -> int:
    return engine.run_until_done(max_iterations if max_iterations > 0 else None)


def cancel(engine: Engine, request_id: int) -> int:
    return int(engine.cancel(request_id))


def request(engine: Engine, request_id: int) -> Tuple[int, str, int, int, int, int, str]:
    """(state index, stop reason, prompt tokens, generated tokens, tokens in the cache,
    preemptions, error text)."""
    item = engine.request(request_id)
    cached = engine.cache.length(request_id) if engine.cache.has(request_id) \
        else engine.cached_at_finish(request_id)
    return (STATES.index(item.state.value), item.stop_reason.value if item.stop_reason else "",
            len(item.prompt), len(item.generated), cached, item.preemptions, item.error or "")


def generated(engine: Engine, request_id: int) -> List[int]:
    return list(engine.request(request_id).generated)


def stats(engine: Engine) -> Tuple[int, int, int, int, int, int, int, int, int, int]:
    """(iterations, prefill tokens, decode tokens, finished, cancelled, failed, preemptions,
    steps run, free pages, pages)."""
    report = engine.stats()
    scheduler, groups = report["scheduler"], report["cache"]["groups"]
    return (scheduler["iterations"], scheduler["prefill_tokens"], scheduler["decode_tokens"],
            scheduler["finished"], scheduler["cancelled"], scheduler["failed"],
            scheduler["preemptions"], report["steps"],
            min((group["free_pages"] for group in groups), default=0),
            min((group["pages"] for group in groups), default=0))


def metrics(engine: Engine) -> Tuple[float, ...]:
    """Counts and rates, then P50 and P95 of the time to the first token and of the time
    between tokens (seconds)."""
    seen = engine.metrics()
    return (float(seen.request_count), float(seen.finished_count), float(seen.failed_count),
            float(seen.prompt_tokens_processed), float(seen.generated_tokens),
            seen.observation_seconds, seen.generated_tokens_per_second,
            seen.time_to_first_token.p50_seconds, seen.time_to_first_token.p95_seconds,
            seen.inter_token_latency.p50_seconds, seen.inter_token_latency.p95_seconds)
