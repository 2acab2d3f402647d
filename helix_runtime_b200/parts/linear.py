"""Matrix products of the parts: ``out (op)= x @ w.T`` with ``w`` stored ``[out, in]``.

bfloat16 goes to the tcgen05 kernel whenever it takes the shape, otherwise (and always in
float32) to the CUDA-core kernel; the choice depends on the shape and the dtype only, never
on a setting.

Weight streaming.  With few tokens (decoding) a product is a pure stream of its weight
matrix, and a matrix has too few 128-row tiles to keep every SM loading: 96 tiles for the
fused QKV matrix of a 4096-wide model, 32 for the output projection, on a GPU of 148 SMs.  Such products are cut
along the reduction as well (split-K) into a few hundred work units that sum into a float32
accumulator with atomic adds.  The residual stream is such an accumulator already; for the
products whose result is stored in bfloat16 (QKV, gate/up) the accumulator is a small
scratch buffer that the NEXT kernel (rotary encoding, SwiGLU) reads, rounds exactly as the
product's own store would have, and clears again.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import library as ops

# At most this many tokens: the product is a weight stream.  (Measured on whole steps of the
# Llama-2-7B sizes: a prompt portion of 65, 96 and 128 tokens takes 3.9, 4.0 and 4.2 ms this
# way against 5.4, 5.6 and 5.8 ms through the tiles of the prompt kernel, of which so few
# tokens make fewer than there are SMs; from 192 tokens on the prompt kernel wins.)
STREAMING_MAX_TOKENS = 128
WAVE_FILL = 0.8                # share of the CTA slots of one wave that a weight stream takes
MIN_K_BLOCKS = 8               # 64-wide reduction blocks per unit, at least


class Weight:
    """A matrix ``[out, in]`` held the way its product kernel reads it best.

    bfloat16 matrices whose depth the tensor-core kernel takes are stored as tiles (every
    [128 x 64] box the kernel loads is 16 contiguous kilobytes, so a product that streams its
    weights once reads DRAM in long runs); ``tile=False`` keeps such a matrix row-major (the
    fused gate/up matrix needs that when the up rows do not start on a tile).  Everything else
    (float32, depths that are no multiple of 8) stays row-major for the CUDA-core kernel."""

    def __init__(self, matrix: torch.Tensor, tile: bool = True) -> None:
        if matrix.dim() != 2:
            raise ValueError("a weight is a matrix")
        self.rows, self.depth = int(matrix.shape[0]), int(matrix.shape[1])
        self.dtype = matrix.dtype
        self.tensor_cores = (matrix.dtype == torch.bfloat16 and matrix.is_cuda and
                             ops.gemm_tc_supports(1, self.rows, self.depth, self.depth, self.depth))
        self.tiles: Optional[torch.Tensor] = None
        self.matrix: Optional[torch.Tensor] = None
        if self.tensor_cores and tile:
            self.tiles = ops.tile_weights(matrix)
        else:
            self.matrix = matrix.contiguous()

    @property
    def shape(self):
        return (self.rows, self.depth)

    def nbytes(self) -> int:
        held = self.tiles if self.tiles is not None else self.matrix
        return held.numel() * held.element_size()


def uses_tensor_cores(x: torch.Tensor, w: Weight, tokens: int) -> bool:
    return (w.tensor_cores and x.dtype == torch.bfloat16 and tokens > 0 and
            x.stride(0) % 8 == 0)


def _gemm_tc(x, w: Weight, out, tokens, features, epilogue, status, **options) -> None:
    if w.tiles is not None:
        ops.gemm_tc(x, w.tiles, out, tokens, features, epilogue, status, weight_shape=w.shape,
                    **options)
    else:
        ops.gemm_tc(x, w.matrix, out, tokens, features, epilogue, status, **options)


def _gemm_simt(x, w: Weight, out, tokens, epilogue) -> None:
    if w.matrix is None:
        raise RuntimeError("this product needs the CUDA-core kernel, but the weight is held as "
                           "tiles for the tensor cores")
    ops.gemm_simt(x, w.matrix, out, tokens, epilogue)


def is_weight_stream(x: torch.Tensor, w: Weight, tokens: int) -> bool:
    return tokens <= STREAMING_MAX_TOKENS and uses_tensor_cores(x, w, tokens)


def split_k_for(tokens: int, features: int, depth: int, ordered: bool = False) -> int:
    """Ways to cut the reduction of a weight-streaming product (1: not at all).  ``ordered``:
    the caller wants sums in a fixed order, which atomic adds of several splits cannot give.

    A product of few tokens has too few 128-row tiles to keep every SM loading, so its tiles
    are cut along the reduction until the CTAs fill ONE wave to about four fifths (two CTAs
    share an SM): every CTA then starts at once, each
    ends with one round of atomic adds, and the slots left over take the CTAs of the NEXT
    kernel, which is let in early and fetches its first weights meanwhile.  Measured on whole
    decode steps of the Llama-2-7B sizes against cutting into four units per SM (two waves):
    batch 1, 4, 8: 4 % less time (2.87 -> 2.75, 3.10 -> 2.98, 3.29 -> 3.16 ms), batch 16:
    2 % less.  A wave filled to the brim (the fused QKV matrix cut three ways: 288 CTAs on 296
    slots) costs 3 % at batch 8 and 13 % at batch 16, and a wave and a bit is as bad."""
    if tokens > STREAMING_MAX_TOKENS or ordered:
        return 1
    tiles = -(-features // 128)
    k_blocks = -(-depth // 64)
    splits = int(WAVE_FILL * 2 * ops.sm_count()) // tiles
    return max(1, min(splits, k_blocks // MIN_K_BLOCKS))


def project(x: torch.Tensor, w: Weight, out: torch.Tensor, tokens: int, epilogue: int,
            status: torch.Tensor, ordered: bool = False) -> None:
    """``out[:tokens] (op)= x[:tokens] @ w.T``; epilogue is one of ops.EPI_STORE,
    ops.EPI_STORE_F32, ops.EPI_ADD_F32.  ``ordered``: no split-K (see ``split_k_for``)."""
    if tokens == 0:
        return
    if uses_tensor_cores(x, w, tokens):
        splits = split_k_for(tokens, w.rows, w.depth, ordered) \
            if epilogue == ops.EPI_ADD_F32 else 1
        _gemm_tc(x, w, out, tokens, w.rows, epilogue, status, k_splits=splits)
    else:
        _gemm_simt(x, w, out, tokens, epilogue)


def project_into_accumulator(x: torch.Tensor, w: Weight, accumulator: torch.Tensor,
                             tokens: int, status: torch.Tensor, ordered: bool = False) -> None:
    """``accumulator[:tokens] += x[:tokens] @ w.T`` as a split-K weight stream (float32; the
    accumulator is clear on entry and its reader clears it again)."""
    splits = split_k_for(tokens, w.rows, w.depth, ordered)
    _gemm_tc(x, w, accumulator, tokens, w.rows, ops.EPI_ADD_F32, status, k_splits=splits)


def project_swiglu(x: torch.Tensor, w_gate_up: Weight, intermediate: int, act: torch.Tensor,
                   workspace, capacity: int, tokens: int, status: torch.Tensor,
                   ordered: bool = False) -> None:
    """``act[:tokens] = silu(x @ gate.T) * (x @ up.T)`` with ``w_gate_up = [gate; up]``.

    Three routes, one rounding each (float32 gate and up, float32 activation, one store):
    many tokens on the tensor cores: SwiGLU is the product's epilogue; few tokens on the
    tensor cores: split-K into a float32 accumulator, then the SwiGLU kernel, which clears
    it; otherwise the CUDA-core product stores float32 and the SwiGLU kernel follows."""
    if tokens == 0:
        return
    if is_weight_stream(x, w_gate_up, tokens):
        accumulator = workspace.accumulator("mlp.gate_up", (STREAMING_MAX_TOKENS, 2 * intermediate))
        project_into_accumulator(x, w_gate_up, accumulator, tokens, status, ordered)
        ops.swiglu(accumulator[:tokens], act[:tokens], zero_input=True)
    elif uses_tensor_cores(x, w_gate_up, tokens):
        _gemm_tc(x, w_gate_up, act, tokens, intermediate, ops.EPI_SWIGLU, status,
                 up_row_offset=intermediate)
    else:
        scratch = workspace.get("mlp.gate_up", (capacity, 2 * intermediate), torch.float32)
        _gemm_simt(x, w_gate_up, scratch, tokens, ops.EPI_STORE_F32)
        ops.swiglu(scratch[:tokens], act[:tokens])
