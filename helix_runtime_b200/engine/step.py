"""The step function: one batch of (request, its next tokens) through the model.

A step holds, for every request in it, the next tokens of that request: a portion of
a prompt (cut anywhere) or a single decoded token.  All of them run as ONE flattened
batch against the cache that earlier steps left, and the logits at the wanted
positions come back.  The reference has no such function; its engine runs the work
items of an iteration one after the other (src/runtime/cpu_engine.cpp:344-361).

Transaction: pages are reserved before the launch and lengths are published after
it; if anything raises, reserved pages go back and no length moves
(src/runtime/cpu_engine.cpp:191, 207, 235).
"""
from __future__ import annotations

import dataclasses
from typing import Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..models.decoder import DecoderModel
from ..ops import library as ops
from ..parts.base import StepContext, Workspace


@dataclasses.dataclass
class StepEntry:
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()          # places among ``tokens`` whose logits are asked for


class StepError(RuntimeError):
    """The batch is not runnable (bad token, too long, unknown request) or a kernel failed."""


class StepFunction:
    def __init__(self, model: DecoderModel, cache: CacheManager, max_tokens: int,
                 max_requests: int, attention_split_keys: int = 256,
                 ordered_sums: bool = False) -> None:
        if model.device is None:
            raise StepError("the model has no weights bound")
        self.model = model
        self.cache = cache
        self.device = model.device
        self.dtype = model.dtype
        self.max_tokens = int(max_tokens)
        self.max_requests = int(max_requests)
        self.attention_split_keys = int(attention_split_keys)
        self.ordered_sums = bool(ordered_sums)
        self.workspace = Workspace(self.device)
        cap, req = self.max_tokens, self.max_requests
        # one packed int32 block: a single host-to-device copy per step
        self._layout = {}
        cursor = 0
        for name, size in (("token_ids", cap), ("positions", cap), ("token_request", cap),
                           ("want_rows", cap), ("request_slot", req), ("request_start", req + 1),
                           ("request_context", req), ("feed_rows", req)):
            self._layout[name] = (cursor, cursor + size)
            cursor += size
        pin = self.device.type == "cuda"
        self._host = torch.zeros(cursor, dtype=torch.int32, pin_memory=pin)
        self._host_np = self._host.numpy()
        self._device = torch.zeros(cursor, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._uploaded = torch.cuda.Event() if pin else None
        self.last_context: Optional[StepContext] = None
        self.steps_run = 0
        self.tokens_run = 0

    def _view(self, name: str, device: bool):
        begin, end = self._layout[name]
        return (self._device if device else self._host_np)[begin:end]

    # --------------------------------------------------------------------- run

    @property
    def upload_bytes(self) -> int:
        """Bytes of the packed batch description that every step copies to the device."""
        return self._host.numel() * self._host.element_size()

    @property
    def feed_rows(self) -> torch.Tensor:
        """Device view of the rows named by ``prepare(..., feed_rows=...)``."""
        return self._view("feed_rows", True)

    def prepare(self, entries: Sequence[StepEntry], context_hint: int = 0,
                feed_rows: Optional[Sequence[int]] = None):
        """Validate, reserve pages, fill and upload the batch description.
        Returns ``(context, want_rows_device, n_want, new_lengths)``.  ``context_hint`` raises
        the context length that launches are sized for (a caller that will replay the step
        while the requests grow passes the length they will reach).  ``feed_rows``: the step
        is prepared before the host knows its tokens; every entry brings one placeholder token
        and names the row of the previous step's sampled tokens that the device puts in its
        place (:func:`helix_runtime_b200.ops.library.feed_tokens`)."""
        if not entries:
            raise StepError("a step needs at least one entry")
        if len(entries) > self.max_requests:
            raise StepError(f"{len(entries)} requests in one step, at most {self.max_requests}")
        total = sum(len(entry.tokens) for entry in entries)
        if feed_rows is not None and (len(feed_rows) != len(entries) or total != len(entries)):
            raise StepError("a step fed on the device has one token and one row per request")
        if total > self.max_tokens:
            raise StepError(f"{total} tokens in one step, at most {self.max_tokens}")
        seen = set()
        vocab = self.model.vocab_size
        for entry in entries:
            if entry.request in seen:
                raise StepError(f"request {entry.request!r} appears twice in one step")
            seen.add(entry.request)
            if not self.cache.has(entry.request):
                raise StepError(f"request {entry.request!r} is not admitted to the cache")
            if len(entry.tokens) == 0:
                raise StepError(f"request {entry.request!r} brings no tokens")
            ids = np.asarray(entry.tokens, dtype=np.int64)
            if ids.ndim != 1 or int(ids.min()) < 0 or int(ids.max()) >= vocab:
                bad = [int(t) for t in ids.reshape(-1) if not 0 <= int(t) < vocab][:1]
                raise StepError(f"token id {bad[0] if bad else '?'} of request {entry.request!r} "
                                f"is outside the vocabulary of {vocab}")
            for place in entry.want:
                if not 0 <= int(place) < len(entry.tokens):
                    raise StepError(f"wanted place {place} of request {entry.request!r} is "
                                    f"outside its {len(entry.tokens)} tokens")
            if self.cache.reserved(entry.request) + len(entry.tokens) > self.model.max_positions:
                raise StepError(f"request {entry.request!r} would exceed the model's "
                                f"{self.model.max_positions} positions")

        if self._uploaded is not None:
            self._uploaded.synchronize()    # the last upload has left the pinned block
        token_ids = self._view("token_ids", False)
        positions = self._view("positions", False)
        token_request = self._view("token_request", False)
        want_rows = self._view("want_rows", False)
        request_slot = self._view("request_slot", False)
        request_start = self._view("request_start", False)
        request_context = self._view("request_context", False)

        new_lengths: List[int] = []
        reserved: List[Tuple[Hashable, int]] = []
        cursor = 0
        n_want = 0
        max_query = 0
        min_query = 1 << 30
        max_context = 0
        try:
            for index, entry in enumerate(entries):
                count = len(entry.tokens)
                # a step still in flight has reserved its positions already: go on from there
                before = self.cache.reserved(entry.request)
                self.cache.extend(entry.request, before + count)
                reserved.append((entry.request, before))
                token_ids[cursor:cursor + count] = np.asarray(entry.tokens, dtype=np.int32)
                positions[cursor:cursor + count] = np.arange(before, before + count, dtype=np.int32)
                token_request[cursor:cursor + count] = index
                request_slot[index] = self.cache.slot(entry.request)
                request_start[index] = cursor
                request_context[index] = before
                for place in entry.want:
                    want_rows[n_want] = cursor + int(place)
                    n_want += 1
                cursor += count
                new_lengths.append(before + count)
                max_query = max(max_query, count)
                min_query = min(min_query, count)
                max_context = max(max_context, before + count)
            request_start[len(entries)] = cursor
            if feed_rows is not None:
                self._view("feed_rows", False)[:len(entries)] = np.asarray(feed_rows, dtype=np.int32)
        except Exception:
            for request, before in reserved:
                self.cache.rollback(request, keep_length=before)
            raise

        self._device.copy_(self._host, non_blocking=True)
        if self._uploaded is not None:
            self._uploaded.record()
        self.cache.sync_tables()
        ctx = StepContext(
            dtype=self.dtype, device=self.device, workspace=self.workspace,
            capacity=self.max_tokens, n_tokens=cursor, n_requests=len(entries),
            token_ids=self._view("token_ids", True), positions=self._view("positions", True),
            token_request=self._view("token_request", True),
            request_slot=self._view("request_slot", True),
            request_start=self._view("request_start", True),
            request_context=self._view("request_context", True),
            status=self.status, max_query_len=max_query, min_query_len=min_query,
            max_context_len=max(max_context, context_hint),
            attention_split_keys=self.attention_split_keys, ordered_sums=self.ordered_sums,
            host_request_slots=[int(v) for v in request_slot[:len(entries)]],
            host_request_starts=[int(v) for v in request_start[:len(entries) + 1]],
            host_request_contexts=[int(v) for v in request_context[:len(entries)]],
            host_query_lengths=[len(entry.tokens) for entry in entries],
        )
        return ctx, self._view("want_rows", True), n_want, new_lengths

    def run(self, entries: Sequence[StepEntry], check_status: bool = True) -> Optional[torch.Tensor]:
        """Run one step.  Returns float32 logits ``[wanted, vocab]`` in the order of the entries
        and of their ``want`` lists (a view that the next step overwrites), or None."""
        ctx, want_rows, n_want, new_lengths = self.prepare(entries)
        try:
            logits = self.model.forward(ctx, self.cache, want_rows, n_want)
            if check_status:
                self.raise_on_status()
        except Exception:
            self.fail(entries)
            raise
        self.finish(entries, new_lengths, ctx)
        return logits

    def finish(self, entries: Sequence[StepEntry], new_lengths: Sequence[int],
               ctx: StepContext) -> None:
        """The step succeeded: publish the new lengths."""
        for entry, length in zip(entries, new_lengths):
            if self.cache.has(entry.request):    # a request may have ended while in flight
                self.cache.commit(entry.request, length)
        self.last_context = ctx
        self.steps_run += 1
        self.tokens_run += ctx.n_tokens

    def fail(self, entries: Sequence[StepEntry],
             keep_lengths: Optional[Sequence[int]] = None, after: Optional[int] = None) -> None:
        """The step failed: give back what was reserved for it; no length moves.
        ``keep_lengths``: what an earlier step that is still in flight has reserved for each
        entry, which stays.  ``after``: a later step, already queued on the device, that may
        still write the pages given back (they are parked until it completes)."""
        self.workspace.clear_accumulators()
        for index, entry in enumerate(entries):
            if self.cache.has(entry.request):
                self.cache.rollback(entry.request,
                                    None if keep_lengths is None else keep_lengths[index],
                                    after=after)

    @staticmethod
    def describe_status(flags: int) -> str:
        names = [name for bit, name in ((ops.FLAG_BAD_TOKEN, "token id outside the vocabulary"),
                                        (ops.FLAG_BAD_PAGE, "block table entry outside the pool"),
                                        (ops.FLAG_WAIT_TIMEOUT, "a bounded kernel wait ran out"),
                                        (ops.FLAG_NONFINITE, "non-finite logits"),
                                        (ops.FLAG_BAD_POSITION,
                                         "a position outside the position table"))
                 if flags & bit]
        return "the step's kernels reported: " + "; ".join(names)

    def raise_on_status(self) -> None:
        """Read the device status word (synchronises) and raise if a kernel flagged a fault."""
        flags = int(self.status.item())
        if flags:
            self.status.zero_()
            raise StepError(self.describe_status(flags))
