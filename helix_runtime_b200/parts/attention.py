"""Causal multi-head attention over the paged cache.

Parameters: ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale`` (default
``1/sqrt(head_dim)``, src/attention/reference.cpp:152), ``window`` (None: all earlier
keys), ``position`` (a position-encoding spec), ``checkpoint_pairing`` (how the
checkpoint's q/k rows are ordered for rotation).  Tensors: ``q``, ``k``, ``v``
``[heads*head_dim, hidden]`` and ``o`` ``[hidden, heads*head_dim]``, all ``[out, in]``.

At load the three projections are fused into one ``[(A + 2 Akv) D, H]`` matrix and,
when the checkpoint rotates half-split pairs while the encoding rotates adjacent
pairs, the rows of q and k are permuted per head to ``[0, D/2, 1, D/2+1, ...]``
(the reference's converter does the same, tools/convert_hf_llama.py:535-542).
Steps: fused projection, rotary encoding + cache append, paged attention, output
projection added into the residual (src/model/cpu_llama.cpp:65-91).

A head whose size is no multiple of 16 (100, say; of 32 above 128) is held in rows of the
next multiple (``row_dim``): the projection gets zero rows for the extra coordinates of every head and
the output projection zero columns, so queries, keys and values carry exact zeros there,
scores and outputs are unchanged, and the tensor-core attention kernels, which tile the
head in steps of 16, take the head.  The scale stays ``1/sqrt(head_dim)`` and the rotation
covers the real coordinates only.  This needs a position encoding that takes a row width
of its own (``row_dim``); with one that does not, the head keeps its size and the
CUDA-core attention runs.
"""
from __future__ import annotations

import math
from typing import List, Mapping, Optional

import torch

from ..cache.manager import KvNeed
from ..config.spec import PartSpec
from ..ops import library as ops
from ..weights.loader import TensorRequest
from .base import LayerCache, Mixer, StepContext, build_part, register_part
from .linear import (STREAMING_MAX_TOKENS, Weight, is_weight_stream, project,
                     project_into_accumulator)


TENSOR_CORE_MIN_QUERY = 16


def row_width(head_dim: int) -> int:
    """The head size the tensor-core attention kernels are built for that holds ``head_dim``:
    steps of 16 up to 128, of 32 up to 256; beyond that the head keeps its size."""
    step = 16 if head_dim <= 128 else 32
    wide = -(-head_dim // step) * step
    return wide if wide <= 256 else head_dim


def rotary_row_permutation(heads: int, head_dim: int, rotary_dim: int) -> torch.Tensor:
    """Row order that turns half-split rotary rows into adjacent-pair rows, per head."""
    half = rotary_dim // 2
    order: List[int] = []
    for head in range(heads):
        base = head * head_dim
        for frequency in range(half):
            order.extend((base + frequency, base + half + frequency))
        order.extend(range(base + rotary_dim, base + head_dim))
    return torch.tensor(order, dtype=torch.long)


class PagedAttention(Mixer):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.heads = int(spec["num_heads"])
        self.kv_heads = int(spec["num_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        if self.heads % self.kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.scale = float(spec.get("scale") or 1.0 / math.sqrt(float(self.head_dim)))
        window = spec.get("window")
        self.window: Optional[int] = int(window) if window else None
        self.row_dim = self.head_dim
        self.position = build_part("position", spec["position"], hidden_size)
        wide = row_width(self.head_dim)
        if wide != self.head_dim:
            position = spec["position"]
            padded = build_part("position", PartSpec(position.kind,
                                                     {**position.params, "row_dim": wide},
                                                     position.tensors), hidden_size)
            if getattr(padded, "row_dim", None) == wide:
                self.position, self.row_dim = padded, wide
        self.checkpoint_pairing = spec.get("checkpoint_pairing", self.position.pairing)
        self.names = dict(spec.tensors)
        # widths of the checkpoint's matrices and of the rows this part computes with
        self.q_rows = self.heads * self.head_dim
        self.kv_rows = self.kv_heads * self.head_dim
        self.q_size = self.heads * self.row_dim
        self.kv_size = self.kv_heads * self.row_dim
        self.qkv_size = self.q_size + 2 * self.kv_size
        self.w_qkv: Optional[Weight] = None
        self.w_o: Optional[Weight] = None

    def kv_need(self) -> Optional[KvNeed]:
        return KvNeed(self.kv_heads, self.row_dim, self.window)

    def tensor_requests(self) -> List[TensorRequest]:
        h = self.hidden_size
        return [
            TensorRequest(self.names["q"], (self.q_rows, h)),
            TensorRequest(self.names["k"], (self.kv_rows, h)),
            TensorRequest(self.names["v"], (self.kv_rows, h)),
            TensorRequest(self.names["o"], (h, self.q_rows)),
            *self.position.tensor_requests(),
        ]

    def widen_rows(self, matrix: torch.Tensor, heads: int) -> torch.Tensor:
        """``[heads * head_dim, in]`` to ``[heads * row_dim, in]``: zero rows behind each head."""
        if self.row_dim == self.head_dim:
            return matrix
        wide = matrix.new_zeros((heads, self.row_dim, matrix.shape[1]))
        wide[:, :self.head_dim] = matrix.reshape(heads, self.head_dim, matrix.shape[1])
        return wide.reshape(heads * self.row_dim, matrix.shape[1])

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        q = tensors[self.names["q"]]
        k = tensors[self.names["k"]]
        v = tensors[self.names["v"]]
        if (self.checkpoint_pairing is not None and self.position.pairing is not None
                and self.checkpoint_pairing != self.position.pairing):
            if self.checkpoint_pairing == "half_split" and self.position.pairing == "adjacent":
                rotary = self.position.rotary_dim
                q = q[rotary_row_permutation(self.heads, self.head_dim, rotary).to(q.device)]
                k = k[rotary_row_permutation(self.kv_heads, self.head_dim, rotary).to(k.device)]
            else:
                raise ValueError(f"no row permutation from {self.checkpoint_pairing!r} to "
                                 f"{self.position.pairing!r}")
        q, k, v = (self.widen_rows(q, self.heads), self.widen_rows(k, self.kv_heads),
                   self.widen_rows(v, self.kv_heads))
        o = self.widen_rows(tensors[self.names["o"]].t().contiguous(), self.heads).t()
        self.w_qkv = Weight(torch.cat([q, k, v], dim=0).to(device=device, dtype=dtype).contiguous())
        self.w_o = Weight(o.to(device=device, dtype=dtype).contiguous())
        self.position.bind(tensors, dtype, device)

    @property
    def graph_safe(self) -> bool:
        return self.position.graph_safe

    def weight_bytes(self) -> int:
        return self.w_qkv.nbytes() + self.w_o.nbytes()

    def split_keys_for(self, tokens: int, longest: int, limit: int) -> int:
        """Keys per split.  One warp walks one (token, head, split); a step with few tokens
        (decoding) gets narrower splits so that about sixteen warps per SM stream the cache,
        a step with many tokens keeps ``limit``.  Splits are multiples of the 32-key chunk,
        so the choice changes the order of float32 sums only."""
        wanted_warps = ops.sm_count() * 16
        splits = max(1, wanted_warps // max(1, tokens * self.heads))
        keys = -(-longest // splits)
        keys = max(32, -(-keys // 32) * 32)
        return min(keys, max(32, limit))

    def forward(self, ctx: StepContext, cache: LayerCache, x: torch.Tensor,
                residual: torch.Tensor) -> None:
        n = ctx.n_tokens
        qkv = ctx.workspace.get("attention.qkv", (ctx.capacity, self.qkv_size), ctx.dtype)
        context = ctx.workspace.get("attention.context", (ctx.capacity, self.q_size), ctx.dtype)
        if is_weight_stream(x, self.w_qkv, n):
            # few tokens: split-K into a float32 accumulator that the rotary kernel reads,
            # rounds as the product's store would have, and clears
            accumulator = ctx.workspace.accumulator("attention.qkv",
                                                    (STREAMING_MAX_TOKENS, self.qkv_size))
            project_into_accumulator(x, self.w_qkv, accumulator, n, ctx.status,
                                     ctx.ordered_sums)
            self.position.apply(ctx, cache, qkv, self.heads, self.kv_heads, accum=accumulator)
        elif not self.position.project_and_apply(ctx, cache, x, self.w_qkv, qkv, self.heads,
                                                 self.kv_heads):
            project(x, self.w_qkv, qkv, n, ops.EPI_STORE, ctx.status)
            self.position.apply(ctx, cache, qkv, self.heads, self.kv_heads)

        window = cache.window or 0
        # prompt portions of at least TENSOR_CORE_MIN_QUERY tokens go to the tensor-core
        # kernel (bfloat16, no window, head sizes it has); the rest, decode tokens above all,
        # to the CUDA-core kernel.  A step may need both.
        tensor_cores = (ctx.dtype == torch.bfloat16 and not window
                        and ctx.max_query_len >= TENSOR_CORE_MIN_QUERY
                        and ops.prefill_attention_supports(self.row_dim, cache.page_size))
        if tensor_cores:
            ops.prefill_attention(qkv, cache.keys, cache.values, ctx.request_start,
                                  ctx.request_context, ctx.request_slot, cache.block_tables,
                                  context, ctx.n_requests, n // 64 + ctx.n_requests, self.heads,
                                  self.kv_heads, self.row_dim, cache.page_size, cache.num_pages,
                                  self.scale, TENSOR_CORE_MIN_QUERY, ctx.status,
                                  query_lengths=ctx.host_query_lengths)
        if not tensor_cores or ctx.min_query_len < TENSOR_CORE_MIN_QUERY:
            longest = ctx.max_context_len if not window else min(ctx.max_context_len, window)
            split_keys = self.split_keys_for(n, longest, ctx.attention_split_keys)
            max_splits = max(1, -(-longest // split_keys))
            floats = ops.attention_scratch_floats(n, self.heads, self.row_dim, max_splits,
                                                  ctx.dtype, cache.page_size, window)
            partial = ctx.workspace.at_least("attention.partial", floats, torch.float32)
            arrivals = ctx.workspace.accumulator("attention.arrivals",
                                                 (ctx.capacity * self.heads,), torch.int32)
            ops.paged_attention(qkv, cache.keys, cache.values, ctx.positions, ctx.token_request,
                                ctx.request_slot, cache.block_tables, context, partial, n,
                                self.heads, self.kv_heads, self.row_dim, cache.page_size,
                                cache.num_pages, window, self.scale, split_keys, max_splits,
                                ctx.status, request_start=ctx.request_start,
                                skip_query_len=TENSOR_CORE_MIN_QUERY if tensor_cores else 0,
                                arrivals=arrivals)
        project(context, self.w_o, residual, n, ops.EPI_ADD_F32, ctx.status, ctx.ordered_sums)


register_part("mixer", "paged_attention", PagedAttention)
