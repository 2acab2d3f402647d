"""Matrix products of the parts: ``out (op)= x @ w.T`` with ``w`` stored ``[out, in]``.

bfloat16 goes to the tcgen05 kernel whenever it takes the shape, otherwise (and always in
float32) to the CUDA-core kernel; the choice depends on the shape and the dtype only, never
on a setting.

Weight streaming.  With few tokens (decoding) a product is a pure stream of its weight
matrix, and a matrix has too few 128-row tiles to keep all 148 SMs loading: 96 tiles for the
fused QKV matrix of a 4096-wide model, 32 for the output projection.  Such products are cut
along the reduction as well (split-K) into a few hundred work units that sum into a float32
accumulator with atomic adds.  The residual stream is such an accumulator already; for the
products whose result is stored in bfloat16 (QKV, gate/up) the accumulator is a small
scratch buffer that the NEXT kernel (rotary encoding, SwiGLU) reads, rounds exactly as the
product's own store would have, and clears again.
"""
from __future__ import annotations

import torch

from ..ops import library as ops

SM_COUNT = 148
STREAMING_MAX_TOKENS = 64      # at most this many tokens: the product is a weight stream
WORK_UNITS = 4 * SM_COUNT      # units a weight stream is cut into (two CTAs share an SM)
MIN_K_BLOCKS = 8               # 64-wide reduction blocks per unit, at least


def uses_tensor_cores(x: torch.Tensor, w: torch.Tensor, tokens: int) -> bool:
    return (x.dtype == torch.bfloat16 and tokens > 0 and
            ops.gemm_tc_supports(tokens, w.shape[0], w.shape[1], x.stride(0), w.stride(0)))


def is_weight_stream(x: torch.Tensor, w: torch.Tensor, tokens: int) -> bool:
    return tokens <= STREAMING_MAX_TOKENS and uses_tensor_cores(x, w, tokens)


def split_k_for(tokens: int, features: int, depth: int) -> int:
    """Ways to cut the reduction of a weight-streaming product (1: not at all)."""
    if tokens > STREAMING_MAX_TOKENS:
        return 1
    tiles = -(-features // 128)
    k_blocks = -(-depth // 64)
    splits = max(1, round(WORK_UNITS / tiles))
    return max(1, min(splits, k_blocks // MIN_K_BLOCKS))


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


def project_into_accumulator(x: torch.Tensor, w: torch.Tensor, accumulator: torch.Tensor,
                             tokens: int, status: torch.Tensor) -> None:
    """``accumulator[:tokens] += x[:tokens] @ w.T`` as a split-K weight stream (float32; the
    accumulator is clear on entry and its reader clears it again)."""
    splits = split_k_for(tokens, w.shape[0], w.shape[1])
    ops.gemm_tc(x, w, accumulator, tokens, w.shape[0], ops.EPI_ADD_F32, status, k_splits=splits)


def project_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, intermediate: int, act: torch.Tensor,
                   workspace, capacity: int, tokens: int, status: torch.Tensor) -> None:
    """``act[:tokens] = silu(x @ gate.T) * (x @ up.T)`` with ``w_gate_up = [gate; up]``.

    Three routes, one rounding each (float32 gate and up, float32 activation, one store):
    many tokens on the tensor cores: SwiGLU is the product's epilogue; few tokens on the
    tensor cores: split-K into a float32 accumulator, then the SwiGLU kernel, which clears
    it; otherwise the CUDA-core product stores float32 and the SwiGLU kernel follows."""
    if tokens == 0:
        return
    if is_weight_stream(x, w_gate_up, tokens):
        accumulator = workspace.accumulator("mlp.gate_up", (STREAMING_MAX_TOKENS, 2 * intermediate))
        project_into_accumulator(x, w_gate_up, accumulator, tokens, status)
        ops.swiglu(accumulator[:tokens], act[:tokens], zero_input=True)
    elif uses_tensor_cores(x, w_gate_up, tokens):
        ops.gemm_tc(x, w_gate_up, act, tokens, intermediate, ops.EPI_SWIGLU, status,
                    up_row_offset=intermediate)
    else:
        scratch = workspace.get("mlp.gate_up", (capacity, 2 * intermediate), torch.float32)
        ops.gemm_simt(x, w_gate_up, scratch, tokens, ops.EPI_STORE_F32)
        ops.swiglu(scratch[:tokens], act[:tokens])
