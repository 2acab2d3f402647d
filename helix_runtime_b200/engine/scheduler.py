"""Requests and the FIFO continuous-batching scheduler.

Policy, after the reference's ``FifoScheduler`` (src/scheduler/fifo_scheduler.cpp:149-304):

* running requests are planned first, in admission order, then the waiting queue
  from its head while fewer than ``max_running_requests`` run; the head is never
  skipped;
* a request in prefill wants the rest of its prompt, a decoding request one token;
  what it gets is cut by the iteration's token budget, by ``max_prefill_chunk``
  (this engine's own knob) and by the pages that are free;
* a request that gets nothing, or less than the budget allowed, because pages ran
  out stops the planning of this iteration (``kv_limited``);
* one iteration is in flight at a time and is completed as a whole; a second one may be
  planned *ahead* of its completion when it is known beforehand who takes part in it
  (``schedule_ahead``: every running request decodes one more token), so that the device
  need not wait for the host between two decode steps.

Sampling happens at the end of the step that produced the logits, so a request's
last token needs no step of its own: a request with prompt P and N new tokens runs
its prompt portions plus N-1 decode steps and writes P + N - 1 cache rows, the
reference's count (src/scheduler/fifo_scheduler.cpp:183-193).

When pages run out.  Nothing is swapped out.  Requests wait for the pages of
requests that finish.  A request that could never fit alone is refused at submit
(src/runtime/cpu_engine.cpp:108-118).  If no request at all can be given work
while some are running (each holds pages another needs), the most recently
admitted running request is preempted: its pages go back, and it returns to the
head of the waiting queue to recompute its prompt plus the tokens it had already
generated.  The reference has no such rule and can stall there; this is decided
here so that the engine always makes progress.
"""
from __future__ import annotations

import dataclasses
import enum
from collections import deque
from typing import Callable, Deque, Dict, List, Optional, Sequence


class RequestState(enum.Enum):
    WAITING = "waiting"
    PREFILL = "prefill"
    DECODING = "decoding"
    FINISHED = "finished"
    CANCELLED = "cancelled"
    FAILED = "failed"


class StopReason(enum.Enum):
    MAX_NEW_TOKENS = "max_new_tokens"
    EOS_TOKEN = "eos_token"
    CONTEXT_LIMIT = "context_limit"
    CANCELLED = "cancelled"
    FAILED = "failed"


class WorkKind(enum.Enum):
    PREFILL = "prefill"
    DECODE = "decode"


@dataclasses.dataclass
class Request:
    id: int
    prompt: List[int]
    max_new_tokens: int
    eos_token: Optional[int] = None
    temperature: float = 0.0
    seed: int = 0
    state: RequestState = RequestState.WAITING
    generated: List[int] = dataclasses.field(default_factory=list)
    processed: int = 0                 # tokens of ``feed`` already in the cache
    stop_reason: Optional[StopReason] = None
    error: Optional[str] = None
    preemptions: int = 0
    created_at: float = 0.0
    first_scheduled_at: Optional[float] = None   # first time the request was given work
    first_token_at: Optional[float] = None
    finished_at: Optional[float] = None
    token_times: List[float] = dataclasses.field(default_factory=list)   # per generated token
    resumed_from: int = 0              # generated tokens that were folded into the prompt
    namespace: Optional[str] = None    # prefix sharing: only prompts of one namespace share
    reused_tokens: int = 0             # tokens taken from the prefix index at (re)admission

    @property
    def feed(self) -> List[int]:
        """Everything the model has to read before it can produce the next new token."""
        return self.prompt + self.generated

    @property
    def prompt_tokens_processed(self) -> int:
        """Prompt tokens whose keys and values are in the cache (reused ones included)."""
        return min(self.processed, len(self.prompt))

    @property
    def latest_event_at(self) -> float:
        """The latest time anything was recorded for the request."""
        return max(self.created_at, self.first_scheduled_at or self.created_at,
                   self.token_times[-1] if self.token_times else self.created_at,
                   self.finished_at or self.created_at)

    @property
    def feed_length(self) -> int:
        return len(self.prompt) + len(self.generated)

    def feed_slice(self, offset: int, count: int) -> List[int]:
        """``feed[offset:offset + count]`` without building the whole list."""
        prompt_tokens = len(self.prompt)
        end = offset + count
        if end <= prompt_tokens:
            return self.prompt[offset:end]
        if offset >= prompt_tokens:
            return self.generated[offset - prompt_tokens:end - prompt_tokens]
        return self.prompt[offset:] + self.generated[:end - prompt_tokens]

    @property
    def remaining_feed(self) -> int:
        return len(self.prompt) + len(self.generated) - self.processed

    @property
    def remaining_generation(self) -> int:
        return self.max_new_tokens - len(self.generated)

    @property
    def is_terminal(self) -> bool:
        return self.state in (RequestState.FINISHED, RequestState.CANCELLED, RequestState.FAILED)


@dataclasses.dataclass(frozen=True)
class ScheduledWork:
    request_id: int
    kind: WorkKind
    token_offset: int          # position of the first token of this portion
    token_count: int
    samples: bool              # the portion ends at the request's last fed token: sample after it


@dataclasses.dataclass
class IterationBatch:
    id: int
    work: List[ScheduledWork]
    scheduled_tokens: int = 0
    kv_limited: bool = False
    budget_exhausted: bool = False
    preempted: List[int] = dataclasses.field(default_factory=list)


@dataclasses.dataclass(frozen=True)
class WorkCompletion:
    request_id: int
    ok: bool
    token: Optional[int] = None     # the sampled token when the work item sampled
    error: Optional[str] = None


@dataclasses.dataclass(frozen=True)
class SchedulerConfig:
    max_tokens_per_iteration: int
    max_running_requests: int
    max_prefill_chunk: Optional[int] = None
    # A prompt portion never runs across the prompt's last page boundary, so that some step
    # ends exactly there: what a model keeps per request beside its pages can then be copied
    # as it stands at the end of the prompt's longest page-aligned prefix.
    cut_prompt_at_last_page: bool = False

    def __post_init__(self) -> None:
        if self.max_tokens_per_iteration <= 0 or self.max_running_requests <= 0:
            raise ValueError("scheduler limits must be positive")
        if self.max_prefill_chunk is not None and self.max_prefill_chunk <= 0:
            raise ValueError("max_prefill_chunk must be positive")


class PageLedger:
    """What the scheduler needs to know of the cache: how far a request can grow.

    The engine passes its cache manager (which has these methods); scheduler tests pass
    a fake."""

    def free_pages(self) -> List[int]:
        raise NotImplementedError

    def max_extend(self, request: int, desired: int, available: Sequence[int]) -> int:
        raise NotImplementedError

    def max_extend_new(self, desired: int, available: Sequence[int]) -> int:
        raise NotImplementedError

    def pages_to_extend(self, request: int, new_length: int) -> List[int]:
        raise NotImplementedError


class FifoScheduler:
    def __init__(self, config: SchedulerConfig, page_size: int) -> None:
        self.config = config
        self.page_size = page_size
        self.requests: Dict[int, Request] = {}
        self.waiting: Deque[int] = deque()
        self.running: List[int] = []
        self.active: Optional[IterationBatch] = None
        self.ahead: Optional[IterationBatch] = None      # planned before ``active`` completed
        self._next_request = 0
        self._next_iteration = 0
        self.stats = {"iterations": 0, "prefill_tokens": 0, "decode_tokens": 0,
                      "kv_limited_iterations": 0, "preemptions": 0, "finished": 0,
                      "cancelled": 0, "failed": 0}

    # ------------------------------------------------------------------ submit

    def submit(self, prompt: Sequence[int], max_new_tokens: int, eos_token: Optional[int] = None,
               temperature: float = 0.0, seed: int = 0, now: float = 0.0,
               namespace: Optional[str] = None) -> int:
        if len(prompt) == 0:
            raise ValueError("a request needs at least one prompt token")
        if max_new_tokens < 0:
            raise ValueError("max_new_tokens must not be negative")
        if temperature < 0.0:
            raise ValueError("temperature must not be negative")
        request = Request(id=self._next_request, prompt=[int(t) for t in prompt],
                          max_new_tokens=int(max_new_tokens), eos_token=eos_token,
                          temperature=float(temperature), seed=int(seed), created_at=now,
                          namespace=namespace)
        self._next_request += 1
        self.requests[request.id] = request
        self.waiting.append(request.id)
        return request.id

    def request(self, request_id: int) -> Request:
        return self.requests[request_id]

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    # ---------------------------------------------------------------- schedule

    def schedule_iteration(self, ledger: PageLedger,
                           admit: Callable[[int], None],
                           release: Callable[[int], None],
                           reusable: Optional[Callable[[Request], int]] = None,
                           reclaim: Optional[Callable[[], bool]] = None,
                           now: float = 0.0) -> Optional[IterationBatch]:
        """Plan one iteration.  ``admit(id)`` / ``release(id)`` let the caller give a request
        its cache slot when it starts and take its pages back when it is preempted.
        ``reusable(request)`` says how many leading tokens admission will find in the cache
        already (a shared prefix; whole pages), which then count as progress
        (src/scheduler/fifo_scheduler.cpp:229-239).  ``reclaim()`` is asked for pages when
        nobody can move, before anybody is preempted (the reference's engine evicts prefix
        anchors there, src/runtime/cpu_engine.cpp:323-331); True means: plan again."""
        if self.active is not None:
            raise RuntimeError("an iteration is already in flight")
        preempted: List[int] = []
        while True:
            batch = self._plan(ledger, admit, reusable)
            if batch.work:
                break
            if reclaim is not None and (self.running or self.waiting) and reclaim():
                continue
            if not self.running:
                break
            # nobody can move and somebody holds pages: preempt the youngest running request
            victim = self.running.pop()
            request = self.requests[victim]
            release(victim)
            request.state = RequestState.WAITING
            request.processed = 0
            request.preemptions += 1
            self.waiting.appendleft(victim)
            preempted.append(victim)
            self.stats["preemptions"] += 1
        batch.preempted = preempted
        if not batch.work:
            if batch.kv_limited:
                self.stats["kv_limited_iterations"] += 1
            return None
        self.active = batch
        self.stats["iterations"] += 1
        if batch.kv_limited:
            self.stats["kv_limited_iterations"] += 1
        for work in batch.work:
            key = "prefill_tokens" if work.kind is WorkKind.PREFILL else "decode_tokens"
            self.stats[key] += work.token_count
            request = self.requests[work.request_id]
            if request.first_scheduled_at is None:
                request.first_scheduled_at = max(now, request.created_at)
        return batch

    def schedule_ahead(self, ledger: PageLedger, max_positions: int) -> Optional[IterationBatch]:
        """Plan the iteration after the one in flight before that one's tokens are known, or
        return None when its make-up depends on them.

        It is planned when the iteration in flight decodes one token for every running
        request, none of them can end in it by its count of new tokens or by the context
        limit, nobody waits who could be admitted, and every request has a page for one more
        token.  What cannot be known is an end-of-sequence token: a request that samples one
        in the iteration in flight retires there, and its row of the iteration planned ahead
        is computed for nothing and dropped at completion (as for a request cancelled in
        flight).  The reference completes every iteration before it plans the next
        (src/scheduler/fifo_scheduler.cpp:149-304); this is this engine's own."""
        batch = self.active
        if batch is None or self.ahead is not None:
            return None
        if self.waiting and len(self.running) < self.config.max_running_requests:
            return None
        if len(self.running) > self.config.max_tokens_per_iteration:
            return None
        if [work.request_id for work in batch.work] != self.running:
            return None
        available = list(ledger.free_pages())
        work_ahead: List[ScheduledWork] = []
        for work in batch.work:
            request = self.requests[work.request_id]
            if (work.kind is not WorkKind.DECODE or not work.samples or work.token_count != 1
                    or request.is_terminal or request.remaining_generation < 2
                    or request.processed + 2 > max_positions):
                return None
            if ledger.max_extend(request.id, 1, available) < 1:
                return None
            needed = ledger.pages_to_extend(request.id, request.processed + 2)
            for index, count in enumerate(needed):
                available[index] -= count
            work_ahead.append(ScheduledWork(request_id=request.id, kind=WorkKind.DECODE,
                                            token_offset=request.processed + 1, token_count=1,
                                            samples=True))
        self.ahead = IterationBatch(id=batch.id + 1, work=work_ahead,
                                    scheduled_tokens=len(work_ahead))
        self.stats["iterations"] += 1
        self.stats["decode_tokens"] += len(work_ahead)
        return self.ahead

    def _plan(self, ledger: PageLedger, admit: Callable[[int], None],
              reusable: Optional[Callable[[Request], int]] = None) -> IterationBatch:
        batch = IterationBatch(id=self._next_iteration, work=[])
        remaining_tokens = self.config.max_tokens_per_iteration
        available = list(ledger.free_pages())
        stop = False

        def plan(request: Request, waiting: bool) -> bool:
            nonlocal remaining_tokens, stop
            prefill = waiting or request.state is RequestState.PREFILL
            start = request.processed
            if waiting and reusable is not None:
                start = reusable(request)
                if start % self.page_size != 0 or not 0 <= start < request.feed_length:
                    raise ValueError("a reused prefix is whole pages and leaves a token to run")
            desired = request.feed_length - start
            assert desired > 0, "an active request always has something to feed"
            if prefill and self.config.max_prefill_chunk is not None:
                desired = min(desired, self.config.max_prefill_chunk)
            if prefill and self.config.cut_prompt_at_last_page:
                boundary = len(request.prompt) // self.page_size * self.page_size
                if start < boundary < start + desired:
                    desired = boundary - start
            budgeted = min(desired, remaining_tokens)
            if waiting:
                granted = ledger.max_extend_new(budgeted, available)
            else:
                granted = ledger.max_extend(request.id, budgeted, available)
            if granted == 0:
                batch.kv_limited = True
                stop = True
                return False
            if waiting:
                admit(request.id)
                request.processed = start
                request.reused_tokens = start
            needed = ledger.pages_to_extend(request.id, request.processed + granted)
            for index, count in enumerate(needed):
                available[index] -= count
            batch.work.append(ScheduledWork(
                request_id=request.id,
                kind=WorkKind.PREFILL if prefill else WorkKind.DECODE,
                token_offset=request.processed, token_count=granted,
                samples=granted == request.remaining_feed))
            batch.scheduled_tokens += granted
            remaining_tokens -= granted
            if granted < budgeted:
                batch.kv_limited = True
                stop = True
            elif remaining_tokens == 0:
                batch.budget_exhausted = True
                stop = True
            return True

        for request_id in list(self.running):
            if stop:
                break
            plan(self.requests[request_id], waiting=False)
        while (not stop and self.waiting
               and len(self.running) < self.config.max_running_requests):
            request = self.requests[self.waiting[0]]
            if not plan(request, waiting=True):
                break
            self.waiting.popleft()
            request.state = RequestState.PREFILL
            self.running.append(request.id)
        return batch

    # ---------------------------------------------------------------- complete

    def complete_iteration(self, batch_id: int, completions: Sequence[WorkCompletion],
                           max_positions: int, now: float = 0.0) -> List[Request]:
        """Apply the results of the iteration in flight; return the requests that retired.

        Everything is validated before anything changes
        (src/scheduler/fifo_scheduler.cpp:330-384)."""
        batch = self.active
        if batch is None or batch.id != batch_id:
            raise RuntimeError("no such iteration in flight")
        if len(completions) != len(batch.work):
            raise ValueError("one completion per work item, in order")
        for work, completion in zip(batch.work, completions):
            if completion.request_id != work.request_id:
                raise ValueError("completions must follow the order of the work items")
            if completion.ok and work.samples and completion.token is None:
                raise ValueError(f"request {work.request_id} sampled but reports no token")
        retired: List[Request] = []
        for work, completion in zip(batch.work, completions):
            request = self.requests[work.request_id]
            if request.is_terminal:       # cancelled while in flight
                continue
            if not completion.ok:
                self._retire(request, RequestState.FAILED, StopReason.FAILED, now,
                             error=completion.error)
                retired.append(request)
                continue
            request.processed += work.token_count
            if not work.samples:
                continue
            if request.max_new_tokens == 0:
                self._retire(request, RequestState.FINISHED, StopReason.MAX_NEW_TOKENS, now)
                retired.append(request)
                continue
            request.generated.append(int(completion.token))
            request.token_times.append(max(now, request.latest_event_at))
            request.state = RequestState.DECODING
            if request.first_token_at is None:
                request.first_token_at = request.token_times[-1]
            if request.eos_token is not None and completion.token == request.eos_token:
                self._retire(request, RequestState.FINISHED, StopReason.EOS_TOKEN, now)
            elif request.remaining_generation == 0:
                self._retire(request, RequestState.FINISHED, StopReason.MAX_NEW_TOKENS, now)
            elif request.processed >= max_positions:
                self._retire(request, RequestState.FINISHED, StopReason.CONTEXT_LIMIT, now)
            if request.is_terminal:
                retired.append(request)
        self.active, self.ahead = self.ahead, None
        self._next_iteration += 1
        return retired

    def cancel(self, request_id: int, now: float = 0.0) -> bool:
        request = self.requests[request_id]
        if request.is_terminal:
            return False
        self._retire(request, RequestState.CANCELLED, StopReason.CANCELLED, now)
        return True

    def _retire(self, request: Request, state: RequestState, reason: StopReason, now: float,
                error: Optional[str] = None) -> None:
        request.state = state
        request.stop_reason = reason
        request.error = error
        request.finished_at = max(now, request.latest_event_at)
        if request.id in self.running:
            self.running.remove(request.id)
        if request.id in self.waiting:
            self.waiting.remove(request.id)
        self.stats[{RequestState.FINISHED: "finished", RequestState.CANCELLED: "cancelled",
                    RequestState.FAILED: "failed"}[state]] += 1
