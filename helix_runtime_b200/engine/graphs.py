"""CUDA graphs of decode steps: one launch for the whole forward pass and the sampling.

A decode step of a given batch size launches the same few hundred small kernels every time
with the same scalar arguments; only the contents of the step's device buffers change
(token ids, positions, block tables).  Such a step is recorded once into a CUDA graph and
replayed, which removes the launch overhead that otherwise dominates small batches.  The
reference synchronises after every layer (src/model/cuda_llama.cpp:395); here nothing
synchronises inside a step.

A graph is keyed by everything that is baked into its launches: the number of tokens, the
number of wanted rows, the context length attention was launched for (rounded up to a
bucket, so that one graph serves hundreds of consecutive steps), and whether sampling is
greedy.  A key is recorded when it has come up a few times: while requests join one by one,
batch sizes pass that are never seen again.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..parts.base import StepContext


CONTEXT_BUCKET = 256     # decode steps are prepared for a context of this times a power of two
RECORD_AT_USE = 3        # a key is recorded when it comes up for this many times


def bucketed_context(length: int) -> int:
    """The context length a decode step is prepared for: 256, 512, 1024, ...  What is sized by
    it (the bound of the attention's grid, the key splits of the float32 kernel) costs little
    when it is too large, and every bucket is a graph to record."""
    bucket = CONTEXT_BUCKET
    while bucket < length:
        bucket *= 2
    return bucket


class DecodeGraphs:
    def __init__(self, step_function, sampler, max_graphs: int = 64) -> None:
        self.step_function = step_function
        self.sampler = sampler
        self.max_graphs = max_graphs
        self._graphs: Dict[Tuple[int, int, int, bool], torch.cuda.CUDAGraph] = {}
        self._stream = torch.cuda.Stream(device=step_function.device)
        self.replays = 0
        self.captures = 0
        self._uses: Dict[Tuple, int] = {}
        self.kernels_per_graph: Dict[Tuple[int, int, int, bool], int] = {}

    def key_for(self, ctx: StepContext, n_want: int, greedy: bool) -> Tuple[int, int, int, bool]:
        # launches are sized from the token count and the context length the step was
        # prepared for (callers round it up to a bucket, see CONTEXT_BUCKET)
        return (ctx.n_tokens, n_want, ctx.max_context_len, greedy)

    def run(self, ctx: StepContext, want_rows: torch.Tensor, n_want: int, greedy: bool,
            feed_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run the step (forward, then sampling of the wanted rows) and return the device
        tensor of sampled ids.  The first time a key is seen the step runs eagerly and is
        recorded afterwards; from then on it is replayed.  ``feed_rows`` (device, one per
        token): the step's tokens are the ids the previous step sampled in these rows, put in
        place by the first kernel of the graph."""
        from ..ops import library as ops
        key = self.key_for(ctx, n_want, greedy) + (("fed",) if feed_rows is not None else ())
        graph = self._graphs.get(key)
        if graph is not None:
            graph.replay()
            self.replays += 1
            return self.sampler.tokens[:n_want]

        def body() -> torch.Tensor:
            if feed_rows is not None:
                ops.feed_tokens(ctx.token_ids, self.sampler.tokens, feed_rows, ctx.n_tokens)
            logits = self.step_function.model.forward(ctx, self.step_function.cache, want_rows,
                                                      n_want)
            return self.sampler.launch(logits, greedy, ctx.status)

        tokens = body()                      # eager: gives this step's result, sizes workspaces
        self._uses[key] = self._uses.get(key, 0) + 1
        if len(self._graphs) < self.max_graphs and self._uses[key] >= RECORD_AT_USE:
            self._capture(key, body)
        return tokens

    def _capture(self, key, body) -> torch.cuda.CUDAGraph:
        from ..ops import library as ops
        graph = torch.cuda.CUDAGraph()
        current = torch.cuda.current_stream()
        before = ops.launch_count()
        # capture_begin / capture_end directly: the body allocates nothing (the eager run before
        # it has sized every buffer), so the collector run and the emptying of the allocator's
        # cache that the context manager brings along, tens of milliseconds, buy nothing here
        self._stream.wait_stream(current)
        with torch.cuda.stream(self._stream):
            graph.capture_begin()
            try:
                body()
            finally:
                graph.capture_end()
        current.wait_stream(self._stream)
        self.kernels_per_graph[key] = ops.launch_count() - before
        self._graphs[key] = graph
        self.captures += 1
        return graph
