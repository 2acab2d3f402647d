"""Rotary position encoding with the cache append fused into the same kernel.

Parameters: ``theta``, ``head_dim``, ``rotary_dim`` (default: all of the head),
``row_dim`` (default ``head_dim``: the width a head has in the projected rows and in the
cache; the coordinates from ``head_dim`` on are carried along unrotated),
``pairing`` (``adjacent``: pairs ``(2p, 2p+1)`` as the reference rotates,
src/kernels/cpu/reference.cpp:519-531; ``half_split``: pairs ``(p, p + rotary_dim/2)``),
``max_positions``.  The cos/sin table ``[max_positions, rotary_dim/2]`` is built once
in double and cast to float32, as the reference builds its table
(src/model/llama_common.cpp:37-46); the kernel rotates in float32.
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..config.spec import PartSpec
from ..ops import library as ops
from .base import LayerCache, PositionEncoding, StepContext, register_part
from .linear import Weight, uses_tensor_cores

PAIRINGS = {"adjacent": 0, "half_split": 1}


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.theta = float(spec["theta"])
        self.head_dim = int(spec["head_dim"])
        self.rotary_dim = int(spec.get("rotary_dim", self.head_dim))
        self.row_dim = int(spec.get("row_dim", self.head_dim))
        if self.row_dim < self.head_dim:
            raise ValueError("row_dim must be at least head_dim")
        self.max_positions = int(spec["max_positions"])
        pairing = spec.get("pairing", "adjacent")
        if pairing not in PAIRINGS:
            raise ValueError(f"unknown rotary pairing {pairing!r}")
        self.pairing = pairing
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        if not self.theta > 0.0:
            raise ValueError("rotary theta must be positive")
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        half = max(self.rotary_dim // 2, 1)
        # the reference holds theta as a float32 value (include/helix/model/llama.hpp:22)
        theta = float(torch.tensor(self.theta, dtype=torch.float32).item())
        exponent = -2.0 * torch.arange(half, dtype=torch.float64) / float(max(self.rotary_dim, 1))
        frequency = torch.pow(torch.tensor(theta, dtype=torch.float64), exponent)
        angle = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * frequency[None, :]
        self.cos = torch.cos(angle).to(torch.float32).to(device).contiguous()
        self.sin = torch.sin(angle).to(torch.float32).to(device).contiguous()

    def apply(self, ctx: StepContext, cache: LayerCache, qkv: torch.Tensor, heads: int,
              kv_heads: int, accum: Optional[torch.Tensor] = None) -> None:
        """Encode queries and keys of ``qkv[:n_tokens]`` in place; write keys and values into
        the pages when the entry owns its cache.  With ``accum`` the projection is taken from
        that float32 accumulator (and the accumulator cleared) instead of from ``qkv``."""
        write = cache.owns and cache.keys is not None
        ops.rope_append(qkv, ctx.positions, ctx.token_request, ctx.request_slot,
                        cache.block_tables, cache.keys if write else None,
                        cache.values if write else None, self.cos, self.sin, ctx.n_tokens, heads,
                        kv_heads, self.row_dim, self.rotary_dim, PAIRINGS[self.pairing],
                        cache.page_size, cache.num_pages, ctx.status, accum=accum)


    def project_and_apply(self, ctx: StepContext, cache: LayerCache, x: torch.Tensor,
                          weight: Weight, qkv: torch.Tensor, heads: int, kv_heads: int) -> bool:
        """Prompt portions in bfloat16: rotation and cache append are the epilogue of the
        tensor-core product, which saves a pass over the projected rows (read 3 heads' worth,
        write it again) per layer.  Needs adjacent pairs (a thread of the epilogue holds 16
        consecutive coordinates of one token) and heads in steps of 16."""
        n = ctx.n_tokens
        if (self.pairing != "adjacent" or self.row_dim % 16
                or weight.rows != (heads + 2 * kv_heads) * self.row_dim
                or n < ops.gemm_tc_rope_append_min_tokens() or not uses_tensor_cores(x, weight, n)
                or qkv.dtype != torch.bfloat16 or qkv.stride(0) % 8):
            return False
        write = cache.owns and cache.keys is not None
        held = weight.tiles if weight.tiles is not None else weight.matrix
        ops.gemm_tc_rope_append(x, held, qkv, n, ctx.positions, ctx.token_request,
                                ctx.request_slot, cache.block_tables if write else None,
                                cache.keys if write else None, cache.values if write else None,
                                self.cos, self.sin, heads, kv_heads, self.row_dim, self.rotary_dim,
                                cache.page_size, cache.num_pages, ctx.status,
                                weight_shape=weight.shape)
        return True


register_part("position", "rotary", RotaryEncoding)
