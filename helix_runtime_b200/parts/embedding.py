"""Token embedding and the output head.

Embedding: ``hidden[t] = table[id[t]]`` widened into the float32 residual stream
(src/model/cpu_llama.cpp:21-27, 49).  Head: ``logits = x @ head.T`` in float32
(src/model/cpu_llama.cpp:107); when the checkpoint has no head tensor and ties its
embeddings the table stands in (tools/convert_hf_llama.py:497-510).
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..config.spec import PartSpec
from ..ops import library as ops
from ..weights.loader import TensorRequest
from .base import Part, StepContext, register_part
from .linear import Weight, project


class TokenEmbedding(Part):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.vocab_size = int(spec["vocab_size"])
        self.name = spec.tensors["weight"]
        self.table: Optional[torch.Tensor] = None

    def tensor_requests(self) -> List[TensorRequest]:
        return [TensorRequest(self.name, (self.vocab_size, self.hidden_size), role="embedding")]

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        self.table = tensors[self.name].to(device=device, dtype=dtype).contiguous()

    def forward(self, ctx: StepContext, residual: torch.Tensor) -> None:
        ops.embed(self.table, ctx.token_ids[:ctx.n_tokens], residual[:ctx.n_tokens], ctx.status)


class LmHead(Part):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.vocab_size = int(spec["vocab_size"])
        self.name = spec.tensors["weight"]
        self.fallback = spec.tensors.get("tied_to") if spec.get("tied", False) else None
        self.weight: Optional[Weight] = None

    def tensor_requests(self) -> List[TensorRequest]:
        return [TensorRequest(self.name, (self.vocab_size, self.hidden_size),
                              fallback=self.fallback)]

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        self.weight = Weight(tensors[self.name].to(device=device, dtype=dtype).contiguous())

    def weight_bytes(self) -> int:
        return self.weight.nbytes()

    def forward(self, ctx: StepContext, x: torch.Tensor, logits: torch.Tensor, rows: int) -> None:
        project(x, self.weight, logits, rows, ops.EPI_STORE_F32, ctx.status)


register_part("embedding", "token_table", TokenEmbedding)
register_part("lm_head", "linear", LmHead)
