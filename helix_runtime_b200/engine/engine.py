"""The engine: a model, its cache, the step function, the scheduler and the sampler.

This is the Python entry point.  Its surface follows the reference's runtime engine
(``submit / run_iteration / cancel / stats``, include/helix/runtime/cpu_engine.hpp:70-98)
and its one-sequence generator (``generate`` with ``max_new_tokens`` and an optional
``eos_token``; results carry the generated ids, the stop reason and the number of
cached tokens, include/helix/model/generation.hpp:22-63).
"""
from __future__ import annotations

import dataclasses
import os
import time
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch

from ..cache.manager import CacheManager
from ..cache.prefix import PrefixIndex, PrefixMatch
from ..config.registry import architecture_for
from ..models.decoder import DecoderModel
from ..sampling.sampler import Sampler, uniform_for
from ..weights.loader import load_tensors
from ..weights.random_init import random_tensors, write_model_folder
from ..weights.source import open_model
from ..ops import library as ops
from .scheduler import (FifoScheduler, IterationBatch, Request, RequestState, SchedulerConfig,
                        StopReason, WorkCompletion, WorkKind)
from .graphs import DecodeGraphs, bucketed_context
from .metrics import SchedulerMetrics, observe
from .step import StepEntry, StepError, StepFunction

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"unsupported dtype {name}")
        return name
    try:
        return _DTYPES[name]
    except KeyError:
        raise ValueError(f"unsupported dtype {name!r}; use bfloat16 or float32") from None


def require_cuda(device: Union[str, torch.device]) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("this engine runs on an NVIDIA B200 only; there is no CPU path")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available; this engine has no CPU path")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return device


def load_model(model_dir: str, dtype: Union[str, torch.dtype] = "bfloat16",
               device: Union[str, torch.device] = "cuda:0") -> DecoderModel:
    """Build the model that the configuration names and bind the weights.  ``model_dir`` is a
    folder (``config.json`` and safetensors) or a Helix model file (``MODEL.helix``)."""
    dtype = parse_dtype(dtype)
    device = torch.device(device)
    document, source = open_model(model_dir)
    architecture = architecture_for(document)
    config = architecture.config_from_dict(document)
    model = DecoderModel(architecture.build_spec(config))
    model.config = config
    tensors = load_tensors(source, model.tensor_requests(), dtype, device)
    model.bind(tensors, dtype, device)
    return model


def random_model(config, seed: int, dtype: Union[str, torch.dtype] = "bfloat16",
                 device: Union[str, torch.device] = "cuda:0", std: float = 0.02) -> DecoderModel:
    """A model with seeded random weights made directly on the device (no folder): every
    matrix N(0, std), norm weights one.  Used where writing gigabytes to disk would only
    cost time; :func:`write_random_model` is the mode that writes a folder."""
    dtype = parse_dtype(dtype)
    device = torch.device(device)
    architecture = architecture_for(config.to_dict())
    model = DecoderModel(architecture.build_spec(config))
    model.config = config
    generator = torch.Generator(device=device)
    generator.manual_seed(int(seed))
    tensors: Dict[str, torch.Tensor] = {}
    for request in model.tensor_requests():
        if request.role == "scale":
            tensors[request.name] = torch.ones(request.shape, dtype=torch.float32, device=device)
        else:
            value = torch.empty(request.shape, dtype=dtype, device=device)
            value.normal_(0.0, std, generator=generator)
            tensors[request.name] = value
    model.bind(tensors, dtype, device)
    return model


def write_random_model(directory: str, config, seed: int, std: float = 0.02,
                       scale_std: float = 0.0,
                       storage_dtype: Union[str, torch.dtype] = "bfloat16",
                       gains=None) -> None:
    """The random-weights mode: write ``config.json`` and ``model.safetensors``."""
    architecture = architecture_for(config.to_dict())
    model = DecoderModel(architecture.build_spec(config))
    tensors = random_tensors(model.tensor_requests(), seed, std=std, scale_std=scale_std,
                             storage_dtype=parse_dtype(storage_dtype), gains=gains)
    write_model_folder(directory, config.to_dict(), tensors)


@dataclasses.dataclass(frozen=True)
class EngineConfig:
    page_size: int = 16
    num_pages: Optional[int] = None           # default: enough for max_running * max positions
    window_pages: Optional[Dict[int, int]] = None   # window length -> pages of the groups with
                                              # that window (default: num_pages, like the rest)
    cache_memory_fraction: Optional[float] = None   # instead of num_pages: this share of the
                                              # device memory that is free once the weights are
                                              # loaded goes to the cache pool
    max_running_requests: int = 8
    max_tokens_per_iteration: int = 2048
    max_prefill_chunk: Optional[int] = None
    attention_split_keys: int = 256
    poison_free_pages: bool = False           # debugging: fill free pages with NaN
    prefix_cache_entries: int = 0             # > 0: prompts of one namespace share the pages
                                              # of their common beginning (this many prefixes kept)
    prefix_cache_pages: Optional[int] = None  # page references the kept prefixes may hold
                                              # (default: half the pool)
    cuda_graphs: bool = True                  # replay decode-only steps as CUDA graphs
    lookahead: bool = True                    # queue the next decode step before this one's
                                              # tokens have been read (needs cuda_graphs)
    ordered_sums: bool = False                # decode products sum in a fixed order (no split-K
                                              # atomics): logits repeat bit for bit from run to
                                              # run, at the price of slower weight streams


@dataclasses.dataclass
class GenerationResult:
    generated_tokens: List[int]
    stop_reason: str
    cached_token_count: int
    request_id: int = -1


@dataclasses.dataclass
class _Flight:
    """A step that has been queued on the device and not yet completed."""
    batch: IterationBatch
    slot: int                                         # the sampler's result slot it reports to
    entries: List[StepEntry] = dataclasses.field(default_factory=list)
    result: "IterationResult" = None
    ctx: object = None
    n_want: int = 0
    new_lengths: List[int] = dataclasses.field(default_factory=list)
    decode_only: bool = False
    error: Optional[str] = None
    sequence: int = 0                                 # steps are numbered as they are queued
    done: object = None                               # event behind the step's last kernel
    # request -> (tokens, copies of its per-request state as this step leaves it)
    kept_states: Dict[int, Tuple[int, Dict[int, torch.Tensor]]] = \
        dataclasses.field(default_factory=dict)

    def __post_init__(self) -> None:
        self.result = IterationResult()


@dataclasses.dataclass
class IterationResult:
    scheduled_tokens: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    sampled: int = 0
    retired: List[int] = dataclasses.field(default_factory=list)
    preempted: List[int] = dataclasses.field(default_factory=list)
    kv_limited: bool = False
    budget_exhausted: bool = False
    free_pages_before: List[int] = dataclasses.field(default_factory=list)   # per cache group,
    free_pages_after: List[int] = dataclasses.field(default_factory=list)    # around the iteration
    idle: bool = False


class Engine:
    def __init__(self, model: DecoderModel, config: EngineConfig = EngineConfig()) -> None:
        self.model = model
        self.config = config
        device = require_cuda(model.device)
        kv_needs, state_needs = model.cache_needs()
        pages_per_request = -(-model.max_positions // config.page_size)
        num_pages = config.num_pages or pages_per_request * config.max_running_requests
        if config.num_pages is None and config.cache_memory_fraction is not None:
            if not 0.0 < config.cache_memory_fraction <= 1.0:
                raise ValueError("cache_memory_fraction must be in (0, 1]")
            element = torch.empty((), dtype=model.dtype).element_size()
            fixed = dict(config.window_pages or {})      # pools whose size is given
            page_bytes = fixed_bytes = 0
            for need in kv_needs.values():
                layer_page = 2 * need.kv_heads * need.head_dim * element * config.page_size
                if need.window is not None and need.window in fixed:
                    fixed_bytes += layer_page * fixed[need.window]
                else:
                    page_bytes += layer_page
            free_bytes, _ = torch.cuda.mem_get_info(device)
            num_pages = (int(free_bytes * config.cache_memory_fraction) - fixed_bytes) \
                // max(page_bytes, 1)
            if num_pages < 1:
                raise ValueError("cache_memory_fraction leaves no room for a single page")
        self.cache = CacheManager(kv_needs, state_needs, config.page_size, num_pages,
                                  config.max_running_requests, model.max_positions, model.dtype,
                                  device, poison=config.poison_free_pages,
                                  window_slack_pages=1 if config.prefix_cache_entries > 0 else 0,
                                  window_pages=config.window_pages)
        self.step_function = StepFunction(model, self.cache, config.max_tokens_per_iteration,
                                          config.max_running_requests,
                                          config.attention_split_keys, config.ordered_sums)
        self.scheduler = FifoScheduler(
            SchedulerConfig(config.max_tokens_per_iteration, config.max_running_requests,
                            config.max_prefill_chunk,
                            # per-request state is kept for later requests as it stands at
                            # the prompt's last page boundary: a portion must end there
                            cut_prompt_at_last_page=bool(state_needs)
                            and config.prefix_cache_entries > 0), config.page_size)
        self.sampler = Sampler(device, config.max_running_requests)
        # a model with a part that cannot be recorded runs every step eagerly
        self.graphs = DecodeGraphs(self.step_function, self.sampler) \
            if config.cuda_graphs and model.graph_safe else None
        self._cached_at_finish: Dict[int, int] = {}
        self._release_later: List[int] = []
        self.prefix: Optional[PrefixIndex] = None
        if config.prefix_cache_entries > 0:
            self.prefix = PrefixIndex(self.cache, config.prefix_cache_entries,
                                      config.prefix_cache_pages)
        self._matches: Dict[int, PrefixMatch] = {}      # lookups of the iteration being planned
        self._flight: Optional[_Flight] = None          # the step queued ahead, if any
        self._steps_queued = 0                          # sequence number of the next step
        self.steps_queued_ahead = 0

    # ------------------------------------------------------------ construction

    @classmethod
    def from_pretrained(cls, model_dir: str, dtype: Union[str, torch.dtype] = "bfloat16",
                        device: Union[str, torch.device] = "cuda:0",
                        **engine_options) -> "Engine":
        device = require_cuda(device)
        return cls(load_model(model_dir, dtype, device), EngineConfig(**engine_options))

    @classmethod
    def from_random(cls, config, seed: int = 0, dtype: Union[str, torch.dtype] = "bfloat16",
                    device: Union[str, torch.device] = "cuda:0", **engine_options) -> "Engine":
        device = require_cuda(device)
        return cls(random_model(config, seed, dtype, device), EngineConfig(**engine_options))

    # ----------------------------------------------------------------- requests

    def submit(self, prompt: Sequence[int], max_new_tokens: int = 32,
               eos_token: Optional[int] = None, temperature: float = 0.0, seed: int = 0,
               cache_namespace: Optional[str] = "") -> int:
        """Queue a request; refuse what could never run (src/runtime/cpu_engine.cpp:85-119).
        With the prefix index on, requests of the same ``cache_namespace`` share the pages of
        a common beginning; ``None`` keeps a request out of it."""
        vocab = self.model.vocab_size
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("at least one prompt token ID is required")
        for token in prompt:
            if not 0 <= token < vocab:
                raise ValueError(f"prompt token {token} is outside the vocabulary of {vocab}")
        if eos_token is not None and not 0 <= int(eos_token) < vocab:
            raise ValueError(f"eos token {eos_token} is outside the vocabulary of {vocab}")
        if len(prompt) > self.model.max_positions:
            raise ValueError(f"prompt of {len(prompt)} tokens exceeds the model's "
                             f"{self.model.max_positions} positions")
        if max_new_tokens < 0:
            raise ValueError("max_new_tokens must not be negative")
        # the last generated token is never fed back, so it needs no cache row
        rows = min(len(prompt) + max(max_new_tokens - 1, 0), self.model.max_positions)
        for group, pages in zip(self.cache.groups, self.cache.pages_needed_alone(rows)):
            if pages > group.pool.num_pages:
                raise ValueError(f"the request needs {pages} cache pages, the pool has "
                                 f"{group.pool.num_pages}; it could never run")
        return self.scheduler.submit(prompt, max_new_tokens, eos_token, temperature, seed,
                                     now=time.monotonic(),
                                     namespace=cache_namespace if self.prefix is not None else None)

    def cancel(self, request_id: int) -> bool:
        cancelled = self.scheduler.cancel(request_id, now=time.monotonic())
        if cancelled and self.cache.has(request_id):
            self._finish_cache(request_id)
        return cancelled

    def request(self, request_id: int) -> Request:
        return self.scheduler.request(request_id)

    def cached_at_finish(self, request_id: int) -> int:
        """Tokens a request that has ended had in the cache when it ended (0: still running,
        or never admitted)."""
        return self._cached_at_finish.get(request_id, 0)

    def _finish_cache(self, request_id: int) -> None:
        """The request has ended: its pages and slot go back, at once or, while a step that was
        queued ahead may still touch them, when that step has completed."""
        self._cached_at_finish[request_id] = self.cache.length(request_id)
        in_flight = self._flight
        self.cache.release(request_id, after=None if in_flight is None else in_flight.sequence)

    # ------------------------------------------------------------- prefix index

    def _reusable(self, request: Request) -> int:
        """Tokens a request about to be admitted finds in the prefix index."""
        if self.prefix is None or request.namespace is None:
            return 0
        if request.id not in self._matches:
            match = self.prefix.lookup(request.namespace, request.feed)
            if match is None:
                return 0
            self._matches[request.id] = match
        return self._matches[request.id].tokens

    def _admit(self, request_id: int) -> None:
        match = self._matches.pop(request_id, None)
        if match is None:
            self.cache.admit(request_id)
        else:
            self.cache.adopt(request_id, match.anchor, match.tokens)

    def _reclaim(self) -> bool:
        """Pages ran out and nobody can move: drop the coldest kept prefix."""
        self._matches.clear()          # an anchor that was looked up may be the one that goes
        return self.prefix is not None and self.prefix.evict_for_pressure()

    # ---------------------------------------------------------------- iteration

    def run_iteration(self) -> IterationResult:
        """Complete one iteration: schedule a batch, run it as one step, sample, complete, free
        what retired.  With ``lookahead`` the call also queues the decode step that follows
        behind the one it waits for, when the scheduler can plan it before the tokens are
        known, so the device runs the next step while the host reads this one's tokens,
        completes it and plans again; that step is completed by the next call."""
        flight, self._flight = self._flight, None
        if flight is None:
            self._matches.clear()
            batch = self.scheduler.schedule_iteration(self.cache, admit=self._admit,
                                                      release=self.cache.release,
                                                      reusable=self._reusable,
                                                      reclaim=self._reclaim,
                                                      now=time.monotonic())
            if batch is None:
                return IterationResult(idle=True)
            flight = self._launch(batch, None)
        if self.config.lookahead and self.graphs is not None and flight.decode_only \
                and flight.error is None:
            ahead = self.scheduler.schedule_ahead(self.cache, self.model.max_positions)
            if ahead is not None:
                self._flight = self._launch(ahead, flight)
                self.steps_queued_ahead += 1
        return self._complete(flight)

    def _launch(self, batch: IterationBatch, previous: Optional["_Flight"]) -> "_Flight":
        """Queue the batch's step on the device.  ``previous``: the step in flight whose
        sampled tokens this one reads on the device (same requests, one token each)."""
        flight = _Flight(batch=batch, slot=0 if previous is None else 1 - previous.slot,
                         sequence=self._steps_queued)
        self._steps_queued += 1
        result = flight.result
        result.preempted = list(batch.preempted)
        result.kv_limited = batch.kv_limited
        result.budget_exhausted = batch.budget_exhausted
        result.scheduled_tokens = batch.scheduled_tokens
        result.free_pages_before = self.cache.free_pages()
        entries = flight.entries
        temperatures: List[float] = []
        uniforms: List[float] = []
        feed_rows: Optional[List[int]] = None
        if previous is not None:
            row_of = {entry.request: row for row, entry in enumerate(previous.entries)}
            feed_rows = [row_of[work.request_id] for work in batch.work]
        for work in batch.work:
            request = self.scheduler.request(work.request_id)
            # the scheduler counts the tokens a request has fed, the cache the positions it
            # has pages for; the step takes token values from the one and positions from the
            # other, so they must agree (src/runtime/cpu_engine.cpp:165, 223)
            if self.cache.reserved(work.request_id) != work.token_offset:
                flight.error = (f"request {work.request_id}: the scheduler feeds tokens from "
                                f"{work.token_offset}, the cache stands at "
                                f"{self.cache.reserved(work.request_id)}")
                return flight
            if previous is None:
                tokens = request.feed_slice(work.token_offset, work.token_count)
            else:
                tokens = [0]             # the device puts the token of ``previous`` here
            want = [work.token_count - 1] if work.samples and request.max_new_tokens > 0 else []
            entries.append(StepEntry(work.request_id, tokens, want))
            if want:
                temperatures.append(request.temperature)
                uniforms.append(uniform_for(request.seed, len(request.generated)
                                            + (0 if previous is None else 1)))
            if work.kind is WorkKind.PREFILL:
                result.prefill_tokens += work.token_count
            else:
                result.decode_tokens += work.token_count
        step = self.step_function
        flight.decode_only = all(len(entry.tokens) == 1 and len(entry.want) == 1
                                 for entry in entries)
        try:
            hint = 0
            if flight.decode_only and self.graphs is not None:
                hint = bucketed_context(1 + max(self.cache.reserved(e.request) for e in entries))
            flight.ctx, want_rows, flight.n_want, flight.new_lengths = step.prepare(
                entries, context_hint=hint, feed_rows=feed_rows)
            try:
                tokens = None
                if flight.n_want:
                    greedy = self.sampler.prepare(temperatures, uniforms)
                    if self.graphs is not None and flight.decode_only:
                        tokens = self.graphs.run(
                            flight.ctx, want_rows, flight.n_want, greedy,
                            feed_rows=None if feed_rows is None else step.feed_rows)
                    else:
                        logits = self.model.forward(flight.ctx, self.cache, want_rows,
                                                    flight.n_want)
                        tokens = self.sampler.launch(logits, greedy, step.status)
                else:
                    self.model.forward(flight.ctx, self.cache, want_rows, 0)
                self.sampler.fetch(flight.slot, tokens, step.status)
                self._copy_states_at_prefix_ends(flight)
                flight.done = torch.cuda.Event()
                flight.done.record()
            except Exception:
                # what a step still in flight reserved stays; this step's pages go back
                step.fail(entries, [length - len(entry.tokens) for entry, length
                                    in zip(entries, flight.new_lengths)])
                raise
        except StepError as error:
            flight.error = str(error)
        return flight

    def _copy_states_at_prefix_ends(self, flight: "_Flight") -> None:
        """A model with per-request state and the prefix index on: a prompt portion that ends
        at the prompt's last page boundary (the scheduler cuts one there) leaves the state
        that a later request must start from when it adopts that prefix.  It is copied here,
        on the stream, right behind the step and before the next one changes it."""
        if self.prefix is None or not self.cache.states:
            return
        page = self.config.page_size
        for work in flight.batch.work:
            request = self.scheduler.request(work.request_id)
            boundary = len(request.prompt) // page * page
            if (work.kind is WorkKind.PREFILL and request.namespace is not None and boundary > 0
                    and work.token_offset + work.token_count == boundary):
                flight.kept_states[work.request_id] = (
                    boundary, self.cache.snapshot_state(work.request_id))

    def _complete(self, flight: "_Flight") -> IterationResult:
        """Wait for the step's results and apply them."""
        batch, entries, result = flight.batch, flight.entries, flight.result
        step = self.step_function
        completions: List[WorkCompletion] = []
        if flight.error is None:
            sampled, flags = self.sampler.collect(flight.slot, flight.n_want)
            if flags:
                step.status.zero_()
            if flags & ~ops.FLAG_NONFINITE:
                # anything but per-row non-finite logits condemns the whole step, and with it a
                # step that was queued behind it and has read what this one left
                step.fail(entries, after=None if self._flight is None else self._flight.sequence)
                flight.error = StepFunction.describe_status(flags)
                if self._flight is not None:
                    self._flight.error = flight.error
        if flight.error is None:
            step.finish(entries, flight.new_lengths, flight.ctx)
            for request_id, (tokens, snapshot) in flight.kept_states.items():
                if self.cache.has(request_id):
                    self.cache.keep_state(request_id, tokens, snapshot)
            if self.prefix is not None:
                # a request whose LAST prompt portion has just succeeded leaves its longest
                # aligned prefix to later requests (src/runtime/cpu_engine.cpp:136-160)
                for work in batch.work:
                    request = self.scheduler.request(work.request_id)
                    prompt_tokens = len(request.prompt)
                    if (work.kind is WorkKind.PREFILL and request.namespace is not None
                            and not request.is_terminal
                            and work.token_offset < prompt_tokens
                            <= work.token_offset + work.token_count):
                        self.prefix.publish(request.namespace, request.id, request.prompt)
            cursor = 0
            for work, entry in zip(batch.work, entries):
                token = None
                if entry.want:
                    token = sampled[cursor]
                    cursor += 1
                    if token < 0:
                        completions.append(WorkCompletion(
                            work.request_id, False,
                            error="logits contain a non-finite value"))
                        continue
                elif work.samples:
                    token = 0   # max_new_tokens == 0: nothing is sampled, nothing is used
                completions.append(WorkCompletion(work.request_id, True, token=token))
            result.sampled = cursor
        else:
            completions = [WorkCompletion(work.request_id, False, error=flight.error)
                           for work in batch.work]
        # the step is complete on the device (its results have been read; the event behind
        # its last kernel is waited for, which costs nothing by now): what ended while it was
        # queued may be handed out again
        if flight.done is not None:
            flight.done.synchronize()
        self.cache.settle(flight.sequence)
        retired = self.scheduler.complete_iteration(batch.id, completions,
                                                    self.model.max_positions,
                                                    now=time.monotonic())
        for request in retired:
            if self.cache.has(request.id):
                self._finish_cache(request.id)
            result.retired.append(request.id)
        result.free_pages_after = self.cache.free_pages()
        return result

    def run_until_done(self, max_iterations: Optional[int] = None) -> int:
        iterations = 0
        # a step queued ahead is completed even when every request ended in the one before it
        while self.scheduler.has_unfinished() or self._flight is not None:
            outcome = self.run_iteration()
            iterations += 1
            if outcome.idle:
                raise RuntimeError("the scheduler has unfinished requests but can plan no work")
            if max_iterations is not None and iterations >= max_iterations:
                break
        return iterations

    # ----------------------------------------------------------------- generate

    def generate(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]],
                 max_new_tokens: int = 32, eos_token: Optional[int] = None,
                 temperature: float = 0.0, seed: int = 0,
                 cache_namespace: Optional[str] = "") -> List[GenerationResult]:
        """Generate for one prompt or a list of prompts (token ids in, token ids out)."""
        if len(prompts) > 0 and isinstance(prompts[0], int):
            prompts = [prompts]           # a single prompt
        ids = [self.submit(prompt, max_new_tokens, eos_token, temperature, seed + index,
                           cache_namespace)
               for index, prompt in enumerate(prompts)]
        self.run_until_done()
        results = []
        for request_id in ids:
            request = self.scheduler.request(request_id)
            if request.state is RequestState.FAILED:
                raise RuntimeError(f"request {request_id} failed: {request.error}")
            results.append(GenerationResult(
                generated_tokens=list(request.generated),
                stop_reason=request.stop_reason.value if request.stop_reason else "",
                cached_token_count=self.cached_at_finish(request_id),
                request_id=request_id))
        return results

    def metrics(self, observed_at: Optional[float] = None) -> SchedulerMetrics:
        """Counts, rates and latency distributions over every request this engine has seen
        (include/helix/runtime/cpu_engine.hpp:91); times are ``time.monotonic()`` seconds."""
        return observe(self.scheduler.requests.values(),
                                         time.monotonic() if observed_at is None else observed_at)

    def stats(self) -> Dict[str, object]:
        return {"scheduler": dict(self.scheduler.stats), "cache": self.cache.stats(),
                "prefix": dict(self.prefix.stats, entries=len(self.prefix),
                               page_references=self.prefix.page_references)
                if self.prefix is not None else None,
                "steps": self.step_function.steps_run, "tokens": self.step_function.tokens_run,
                "steps_queued_ahead": self.steps_queued_ahead,
                "workspace_bytes": self.step_function.workspace.bytes()}
