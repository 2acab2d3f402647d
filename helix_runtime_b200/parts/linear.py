"""Matrix products of the parts: ``out (op)= x @ w.T`` with ``w`` stored ``[out, in]``.

bfloat16 goes to the tcgen05 kernel whenever it takes the shape, otherwise (and
always in float32) to the CUDA-core kernel; the choice depends on the shape and the
dtype only, never on a setting.  Split-K is used for the residual-add epilogue when
the weight matrix has too few 128-row tiles to keep every SM streaming.
"""
from __future__ import annotations

import torch

from ..ops import library as ops

SM_COUNT = 148


def uses_tensor_cores(x: torch.Tensor, w: torch.Tensor, tokens: int) -> bool:
    return (x.dtype == torch.bfloat16 and tokens > 0 and
            ops.gemm_tc_supports(tokens, w.shape[0], w.shape[1], x.stride(0), w.stride(0)))


def split_k_for(tokens: int, features: int, depth: int) -> int:
    """How many ways to split the reduction so that about one CTA per SM streams weights."""
    token_tile = 16 if tokens <= 16 else 32 if tokens <= 32 else 64 if tokens <= 64 else \
        128 if tokens <= 128 else 256
    ctas = -(-features // 128) * -(-tokens // token_tile)
    k_blocks = -(-depth // 64)
    if ctas >= SM_COUNT // 2 or tokens > 128:
        return 1
    splits = max(1, SM_COUNT // ctas)
    return max(1, min(splits, k_blocks // 8))


def project(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tokens: int, epilogue: int,
            status: torch.Tensor) -> None:
    """``out[:tokens] (op)= x[:tokens] @ w.T``; epilogue is one of ops.EPI_STORE,
    ops.EPI_STORE_F32, ops.EPI_ADD_F32."""
    if tokens == 0:
        return
    if uses_tensor_cores(x, w, tokens):
        splits = split_k_for(tokens, w.shape[0], w.shape[1]) if epilogue == ops.EPI_ADD_F32 else 1
        ops.gemm_tc(x, w, out, tokens, w.shape[0], epilogue, status, k_splits=splits)
    else:
        ops.gemm_simt(x, w, out, tokens, epilogue)


def project_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, intermediate: int, act: torch.Tensor,
                   gate_up_scratch, tokens: int, status: torch.Tensor) -> None:
    """``act[:tokens] = silu(x @ gate.T) * (x @ up.T)`` with ``w_gate_up = [gate; up]``.

    On the tensor cores the activation is the product's epilogue; otherwise the fused
    product is stored as float32 (``gate_up_scratch()`` returns the ``[rows, 2I]`` float32
    buffer) and a second kernel applies SwiGLU, so both paths round once, after the
    activation."""
    if tokens == 0:
        return
    if uses_tensor_cores(x, w_gate_up, tokens):
        ops.gemm_tc(x, w_gate_up, act, tokens, intermediate, ops.EPI_SWIGLU, status,
                    up_row_offset=intermediate)
    else:
        scratch = gate_up_scratch()
        ops.gemm_simt(x, w_gate_up, scratch, tokens, ops.EPI_STORE_F32)
        ops.swiglu(scratch[:tokens], act[:tokens])
