"""Gated feed-forward: ``down(act(gate(x)) * up(x))`` (src/model/cpu_llama.cpp:93-98).

Parameters: ``intermediate_size``, ``activation`` (``silu``).  Tensors: ``gate``, ``up``
``[intermediate, hidden]`` and ``down`` ``[hidden, intermediate]``.  gate and up are
fused into one ``[2I, H]`` matrix at load so that both products read the input once;
on the tensor cores SwiGLU is the epilogue of that product.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..config.spec import PartSpec
from ..ops import library as ops
from ..weights.loader import TensorRequest
from .base import FeedForward, StepContext, register_part
from .linear import Weight, project, project_swiglu


class GatedMlp(FeedForward):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.intermediate = int(spec["intermediate_size"])
        activation = spec.get("activation", "silu")
        if activation != "silu":
            raise ValueError(f"activation {activation!r} has no kernel; only 'silu'")
        self.names = dict(spec.tensors)
        self.w_gate_up: Optional[Weight] = None
        self.w_down: Optional[Weight] = None

    def tensor_requests(self) -> List[TensorRequest]:
        h, i = self.hidden_size, self.intermediate
        return [TensorRequest(self.names["gate"], (i, h)), TensorRequest(self.names["up"], (i, h)),
                TensorRequest(self.names["down"], (h, i))]

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        fused = torch.cat([tensors[self.names["gate"]], tensors[self.names["up"]]],
                          dim=0).to(device=device, dtype=dtype).contiguous()
        # tiles of 128 rows: the up rows begin on one only when the intermediate size allows
        self.w_gate_up = Weight(fused, tile=self.intermediate % ops.WEIGHT_TILE_ROWS == 0)
        self.w_down = Weight(tensors[self.names["down"]].to(device=device, dtype=dtype).contiguous())

    def weight_bytes(self) -> int:
        return self.w_gate_up.nbytes() + self.w_down.nbytes()

    def forward(self, ctx: StepContext, x: torch.Tensor, residual: torch.Tensor) -> None:
        n = ctx.n_tokens
        act = ctx.workspace.get("mlp.act", (ctx.capacity, self.intermediate), ctx.dtype)
        project_swiglu(x, self.w_gate_up, self.intermediate, act, ctx.workspace, ctx.capacity, n,
                       ctx.status, ctx.ordered_sums)
        project(act, self.w_down, residual, n, ops.EPI_ADD_F32, ctx.status, ctx.ordered_sums)


register_part("feed_forward", "gated_mlp", GatedMlp)
