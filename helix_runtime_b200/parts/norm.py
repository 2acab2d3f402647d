"""RMSNorm: ``y = x / sqrt(mean(x^2) + eps) * w`` (src/kernels/cpu/reference.cpp:392-406).

Reads the float32 residual stream, computes in float32, writes the compute dtype.
Parameters: ``eps``; tensors: ``weight`` ``[hidden]``.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..config.spec import PartSpec
from ..ops import library as ops
from ..weights.loader import TensorRequest
from .base import Norm, StepContext, register_part


class RmsNorm(Norm):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.eps = float(spec["eps"])
        if not self.eps > 0.0:
            raise ValueError("RmsNorm eps must be positive")
        self.weight_name = spec.tensors["weight"]
        self.weight: Optional[torch.Tensor] = None

    def tensor_requests(self) -> List[TensorRequest]:
        return [TensorRequest(self.weight_name, (self.hidden_size,), role="scale")]

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        self.weight = tensors[self.weight_name].to(device=device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.hidden_size * 4

    def forward(self, ctx: StepContext, x: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> None:
        count = ctx.n_tokens if n_rows is None else n_rows
        ops.rmsnorm(x, self.weight, out[:count], self.eps, rows)


register_part("norm", "rms", RmsNorm)
