"""Python face of the CUDA kernel library: one function per entry point.

The functions take ``torch`` tensors, check dtypes and contiguity, and pass raw
device pointers plus the current CUDA stream to the C interface.  Nothing here
computes: there is no CPU path and no library stand-in.  If the shared object
cannot be built or loaded the import of this module's :func:`lib` raises.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional, Sequence, Tuple

import torch

from ..csrc import build as _build

HX_F32 = 0
HX_BF16 = 1

EPI_STORE = 0        # compute dtype out
EPI_STORE_F32 = 1    # float32 out
EPI_ADD_F32 = 2      # float32 out += product
EPI_SWIGLU = 3       # tensor-core kernel only

FLAG_BAD_TOKEN = 1
FLAG_BAD_PAGE = 2
FLAG_WAIT_TIMEOUT = 4
FLAG_NONFINITE = 8
FLAG_BAD_POSITION = 16

_c_int = ctypes.c_int
_c_ptr = ctypes.c_void_p
_c_float = ctypes.c_float

_lock = threading.Lock()
_library: Optional[ctypes.CDLL] = None


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or failed to launch."""


def _declare(library: ctypes.CDLL) -> None:
    library.hx_last_error.restype = ctypes.c_char_p
    library.hx_last_error.argtypes = []
    library.hx_abi_version.restype = _c_int
    library.hx_sm_count.restype = _c_int
    library.hx_sm_count.argtypes = []
    library.hx_embed.argtypes = [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr]
    library.hx_rmsnorm.argtypes = [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_float, _c_ptr]
    library.hx_swiglu.argtypes = [_c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr]
    library.hx_rope_append.argtypes = [
        _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int,
        _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
        _c_ptr, _c_ptr, _c_int, _c_ptr]
    library.hx_gemm_simt.argtypes = [_c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int,
                                     _c_int, _c_int, _c_int, _c_ptr]
    library.hx_gemm_tc.argtypes = [_c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_int, _c_ptr, _c_int,
                                   _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr,
                                   _c_ptr]
    library.hx_gemm_tc_rope_append.argtypes = [
        _c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int,
        _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int,
        _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr]
    library.hx_gemm_tc_rope_append.restype = _c_int
    library.hx_gemm_tc_rope_append_min_tokens.argtypes = []
    library.hx_gemm_tc_rope_append_min_tokens.restype = _c_int
    library.hx_gemm_tc_supports.argtypes = [_c_int] * 5
    library.hx_gemm_tc_token_tile.argtypes = [_c_int]
    library.hx_paged_attention.argtypes = [
        _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr,
        _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
        _c_int, _c_float, _c_int, _c_int, _c_ptr, _c_ptr]
    library.hx_prefill_attention.argtypes = [
        _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int,
        _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_ptr, _c_ptr]
    library.hx_prefill_attention.restype = _c_int
    library.hx_prefill_attention_supports.argtypes = [_c_int, _c_int]
    library.hx_prefill_attention_supports.restype = _c_int
    library.hx_prefill_attention_tc.argtypes = library.hx_prefill_attention.argtypes
    library.hx_prefill_attention_tc.restype = _c_int
    library.hx_prefill_attention_tc_supports.argtypes = [_c_int, _c_int]
    library.hx_prefill_attention_tc_supports.restype = _c_int
    library.hx_paged_attention_scratch_floats.restype = ctypes.c_longlong
    library.hx_paged_attention_scratch_floats.argtypes = [_c_int] * 4
    library.hx_paged_attention_scratch_floats_for.restype = ctypes.c_longlong
    library.hx_paged_attention_scratch_floats_for.argtypes = [_c_int] * 7
    library.hx_argmax.argtypes = [_c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr]
    library.hx_sample.argtypes = [_c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr]
    library.hx_set_dependent_launch.argtypes = [_c_int]
    library.hx_set_dependent_launch.restype = None
    library.hx_launch_count.restype = ctypes.c_longlong
    library.hx_launch_count.argtypes = []
    library.hx_feed_tokens.argtypes = [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr]
    library.hx_feed_tokens.restype = _c_int
    library.hx_bounded_wait_check.argtypes = [_c_int, _c_int, _c_ptr, _c_ptr, _c_ptr]
    library.hx_bounded_wait_check.restype = _c_int
    for name in ("hx_embed", "hx_rmsnorm", "hx_swiglu", "hx_rope_append", "hx_gemm_simt",
                 "hx_gemm_tc", "hx_gemm_tc_supports", "hx_gemm_tc_token_tile",
                 "hx_paged_attention", "hx_argmax", "hx_sample"):
        getattr(library, name).restype = _c_int


def lib() -> ctypes.CDLL:
    """Load (building at first use) the kernel library; raise if that is impossible."""
    global _library
    if _library is None:
        with _lock:
            if _library is None:
                path = _build.build()
                library = ctypes.CDLL(path)
                _declare(library)
                _library = library
    return _library


_sm_counts = {}


def sm_count() -> int:
    """Streaming multiprocessors of the current CUDA device, asked of the device once."""
    device = torch.cuda.current_device()
    if device not in _sm_counts:
        count = int(lib().hx_sm_count())
        if count <= 0:
            raise KernelError(lib().hx_last_error().decode("utf-8", "replace"))
        _sm_counts[device] = count
    return _sm_counts[device]


def library_file() -> str:
    lib()
    return _build.library_path()


def _check(code: int) -> None:
    if code != 0:
        raise KernelError(lib().hx_last_error().decode("utf-8", "replace") or f"kernel error {code}")


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return HX_F32
    if dtype == torch.bfloat16:
        return HX_BF16
    raise KernelError(f"unsupported compute dtype {dtype}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  Every launch asks for it, and a step has hundreds of
    launches: the direct accessor costs a fraction of a microsecond where building a
    ``torch.cuda.Stream`` object costs fourteen (measured: 3.6 ms of a 2,048-token step's
    10 ms of host time)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    return None if tensor is None else tensor.data_ptr()


def _need(tensor: torch.Tensor, dtype: torch.dtype, name: str, last_dim_contiguous: bool = True) -> None:
    if not tensor.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")
    if last_dim_contiguous and tensor.dim() > 0 and tensor.stride(-1) != 1:
        raise KernelError(f"{name} must be contiguous in its last dimension")


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> None:
    """out[t] (float32) = table[ids[t]]."""
    _need(ids, torch.int32, "ids")
    _need(out, torch.float32, "out")
    vocab, hidden = table.shape
    tokens = ids.shape[0]
    assert table.is_contiguous() and out.is_contiguous() and out.shape[1] == hidden
    _check(lib().hx_embed(table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(), out.data_ptr(),
                          tokens, hidden, vocab, _ptr(status), _stream()))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * weight; x and weight float32."""
    _need(x, torch.float32, "x")
    _need(weight, torch.float32, "weight")
    assert x.is_contiguous() and out.is_contiguous()
    hidden = x.shape[-1]
    n_rows = out.shape[0]
    if rows is not None:
        _need(rows, torch.int32, "rows")
        assert rows.shape[0] >= n_rows
    else:
        assert x.shape[0] >= n_rows
    _check(lib().hx_rmsnorm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), dtype_code(out.dtype),
                            _ptr(rows), n_rows, hidden, float(eps), _stream()))


def swiglu(gate_up: torch.Tensor, act: torch.Tensor, zero_input: bool = False) -> None:
    """act[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]; gate_up float32, act compute dtype.
    ``zero_input`` clears what was read (gate_up is a split-K accumulator)."""
    tokens, intermediate = act.shape
    _need(gate_up, torch.float32, "gate_up")
    assert act.is_contiguous()
    _check(lib().hx_swiglu(gate_up.data_ptr(), act.data_ptr(), dtype_code(act.dtype), tokens,
                           intermediate, gate_up.stride(0), 1 if zero_input else 0, _stream()))


def rope_append(qkv: torch.Tensor, positions: torch.Tensor, token_request: torch.Tensor,
                request_table_row: torch.Tensor, block_tables: torch.Tensor,
                k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                cos_table: torch.Tensor, sin_table: torch.Tensor, tokens: int, heads: int,
                kv_heads: int, head_dim: int, rotary_dim: int, pairing: int, page_size: int,
                num_pages: int, status: torch.Tensor,
                accum: Optional[torch.Tensor] = None) -> None:
    """Rotate q and k of ``qkv[:tokens]`` in place and write k, v into their pages.  With
    ``accum`` (float32 ``[rows, width]``) the projection is read from there instead, rounded
    to the storage type, and ``accum`` is cleared."""
    write = k_cache is not None
    _check(lib().hx_rope_append(
        qkv.data_ptr(), dtype_code(qkv.dtype), qkv.stride(0), positions.data_ptr(),
        token_request.data_ptr(), request_table_row.data_ptr(), block_tables.data_ptr(),
        block_tables.stride(0), _ptr(k_cache), _ptr(v_cache), 1 if write else 0,
        cos_table.data_ptr(), sin_table.data_ptr(), cos_table.shape[0], tokens, heads, kv_heads,
        head_dim, rotary_dim, pairing, page_size, num_pages, _ptr(status), _ptr(accum),
        0 if accum is None else accum.stride(0), _stream()))


def gemm_tc_supports(tokens: int, features: int, depth: int, ldx: int, ldw: int) -> bool:
    return bool(lib().hx_gemm_tc_supports(tokens, features, depth, ldx, ldw))


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tokens: int, epilogue: int) -> None:
    """out[:tokens] (op)= x[:tokens] @ w.T on the CUDA cores (float32 or bfloat16 storage)."""
    assert x.dtype == w.dtype and x.stride(-1) == 1 and w.stride(-1) == 1 and out.stride(-1) == 1
    features, depth = w.shape
    _check(lib().hx_gemm_simt(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
                              out.stride(0), dtype_code(x.dtype), tokens, features, depth, epilogue,
                              _stream()))


WEIGHT_TILE_ROWS, WEIGHT_TILE_DEPTH = 128, 64


def tile_weights(matrix: torch.Tensor) -> torch.Tensor:
    """``[rows, depth]`` -> ``[ceil(rows / 128), ceil(depth / 64), 128, 64]``, zero padded:
    every [128 x 64] box the tensor-core product loads becomes 16 contiguous kilobytes."""
    rows, depth = matrix.shape
    row_tiles = -(-rows // WEIGHT_TILE_ROWS)
    k_tiles = -(-depth // WEIGHT_TILE_DEPTH)
    padded = torch.zeros((row_tiles * WEIGHT_TILE_ROWS, k_tiles * WEIGHT_TILE_DEPTH),
                         dtype=matrix.dtype, device=matrix.device)
    padded[:rows, :depth] = matrix
    return padded.view(row_tiles, WEIGHT_TILE_ROWS, k_tiles, WEIGHT_TILE_DEPTH) \
        .permute(0, 2, 1, 3).contiguous()


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tokens: int, features: int,
            epilogue: int, status: torch.Tensor, up_row_offset: int = 0, k_splits: int = 1,
            weight_shape: Optional[Tuple[int, int]] = None) -> None:
    """out[:tokens, :features] (op)= x[:tokens] @ w.T on the tensor cores (bfloat16).  ``w``
    is the matrix ``[rows, depth]`` or its tiles from :func:`tile_weights` (then
    ``weight_shape`` gives rows and depth)."""
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    tiled = w.dim() == 4
    if tiled:
        if weight_shape is None:
            raise ValueError("tiled weights need weight_shape=(rows, depth)")
        rows, depth = weight_shape
        if tuple(w.shape) != (-(-rows // WEIGHT_TILE_ROWS), -(-depth // WEIGHT_TILE_DEPTH),
                              WEIGHT_TILE_ROWS, WEIGHT_TILE_DEPTH) or not w.is_contiguous():
            raise ValueError(f"tiles of shape {tuple(w.shape)} do not hold a {rows} x {depth} matrix")
        ldw = 0
    else:
        rows, depth = w.shape
        ldw = w.stride(0)
    _check(lib().hx_gemm_tc(x.data_ptr(), x.stride(0), x.shape[0], w.data_ptr(), ldw, rows,
                            out.data_ptr(), out.stride(0), tokens, features, depth, epilogue,
                            up_row_offset, k_splits, 1 if tiled else 0, status.data_ptr(),
                            _stream()))


def gemm_tc_rope_append_min_tokens() -> int:
    return int(lib().hx_gemm_tc_rope_append_min_tokens())


def gemm_tc_rope_append(x: torch.Tensor, w: torch.Tensor, qkv: torch.Tensor, tokens: int,
                        positions: torch.Tensor, token_request: torch.Tensor,
                        request_table_row: torch.Tensor, block_tables: Optional[torch.Tensor],
                        k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                        cos_table: torch.Tensor, sin_table: torch.Tensor, heads: int,
                        kv_heads: int, head_dim: int, rotary_dim: int, page_size: int,
                        num_pages: int, status: torch.Tensor,
                        weight_shape: Optional[Tuple[int, int]] = None) -> None:
    """The fused QKV product of a prompt portion (more than 64 tokens, bfloat16) with the
    rotary encoding and the cache append as its epilogue: ``qkv[:tokens, :heads * head_dim]``
    receives the rotated queries (the key and value columns of ``qkv`` are NOT written), keys
    (rotated) and values go to their pages.  Adjacent pairs; ``w`` as for :func:`gemm_tc`."""
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    _need(qkv, torch.bfloat16, "qkv")
    tiled = w.dim() == 4
    if tiled:
        if weight_shape is None:
            raise ValueError("tiled weights need weight_shape=(rows, depth)")
        rows, depth = weight_shape
        if tuple(w.shape) != (-(-rows // WEIGHT_TILE_ROWS), -(-depth // WEIGHT_TILE_DEPTH),
                              WEIGHT_TILE_ROWS, WEIGHT_TILE_DEPTH) or not w.is_contiguous():
            raise ValueError(f"tiles of shape {tuple(w.shape)} do not hold a {rows} x {depth} matrix")
        ldw = 0
    else:
        rows, depth = w.shape
        ldw = w.stride(0)
    write = k_cache is not None
    _check(lib().hx_gemm_tc_rope_append(
        x.data_ptr(), x.stride(0), x.shape[0], w.data_ptr(), ldw, rows, qkv.data_ptr(),
        qkv.stride(0), tokens, depth, 1 if tiled else 0, positions.data_ptr(),
        token_request.data_ptr(), request_table_row.data_ptr(),
        _ptr(block_tables) if write else None,
        block_tables.stride(0) if write else 0, _ptr(k_cache), _ptr(v_cache),
        cos_table.data_ptr(), sin_table.data_ptr(), cos_table.shape[0], heads, kv_heads, head_dim,
        rotary_dim, page_size, num_pages, status.data_ptr(), _stream()))


def attention_scratch_floats(tokens: int, heads: int, head_dim: int, max_splits: int,
                             dtype: Optional[torch.dtype] = None, page_size: int = 0,
                             window: int = 0) -> int:
    """Floats of scratch ``paged_attention`` needs; with ``dtype`` and ``page_size`` given, what
    the kernel that will run for them needs (the streaming kernel: a fixed few megabytes)."""
    if dtype is None:
        return int(lib().hx_paged_attention_scratch_floats(tokens, heads, head_dim, max_splits))
    return int(lib().hx_paged_attention_scratch_floats_for(
        dtype_code(dtype), tokens, heads, head_dim, page_size, window, max_splits))


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    positions: torch.Tensor, token_request: torch.Tensor,
                    request_table_row: torch.Tensor, block_tables: torch.Tensor, out: torch.Tensor,
                    partial: Optional[torch.Tensor], tokens: int, heads: int, kv_heads: int,
                    head_dim: int, page_size: int, num_pages: int, window: int, scale: float,
                    split_keys: int, max_splits: int, status: torch.Tensor,
                    request_start: Optional[torch.Tensor] = None, skip_query_len: int = 0,
                    arrivals: Optional[torch.Tensor] = None) -> None:
    """out[t, h*D:(h+1)*D] = attention of query (t, h) over its request's pages.  With
    ``skip_query_len > 0`` tokens of requests that bring at least that many tokens are left
    out (the tensor-core kernel takes them).  The call needs scratch, made here when it is
    not given: ``partial`` (float32, :func:`attention_scratch_floats` elements) and
    ``arrivals`` (int32, one counter per (token, head), zero on entry; the kernel leaves it
    zero)."""
    if arrivals is None:
        arrivals = torch.zeros(max(1, tokens * heads), dtype=torch.int32, device=q.device)
    if partial is None:
        partial = torch.empty(attention_scratch_floats(tokens, heads, head_dim, max_splits,
                                                       q.dtype, page_size, window),
                              dtype=torch.float32, device=q.device)
    _check(lib().hx_paged_attention(
        q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), dtype_code(q.dtype),
        positions.data_ptr(), token_request.data_ptr(), request_table_row.data_ptr(),
        block_tables.data_ptr(), block_tables.stride(0), _ptr(request_start), skip_query_len,
        out.data_ptr(), out.stride(0),
        _ptr(partial), _ptr(arrivals), tokens, heads, kv_heads, head_dim, page_size, num_pages, window,
        float(scale), split_keys, max_splits, _ptr(status), _stream()))


PREFILL_TILE_ROWS = 64        # query rows of a CTA of the ``mma.sync`` prompt kernel
PREFILL_TILE_ROWS_TC = 256    # and of the tcgen05 prompt kernel


def prefill_attention_supports(head_dim: int, page_size: int) -> bool:
    return bool(lib().hx_prefill_attention_supports(head_dim, page_size))


def prefill_attention_tc_supports(head_dim: int, page_size: int) -> bool:
    return bool(lib().hx_prefill_attention_tc_supports(head_dim, page_size))


def prefill_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      request_start: torch.Tensor, request_context: torch.Tensor,
                      request_table_row: torch.Tensor, block_tables: torch.Tensor,
                      out: torch.Tensor, requests: int, tile_bound: int, heads: int,
                      kv_heads: int, head_dim: int, page_size: int, num_pages: int, scale: float,
                      min_query_len: int, status: torch.Tensor,
                      tensor_memory: Optional[bool] = None,
                      query_lengths: Optional[Sequence[int]] = None) -> None:
    """Tensor-core attention (bfloat16) of every request that brings at least
    ``min_query_len`` tokens; ``tile_bound`` bounds the number of query tiles of 64 tokens
    (the tensor-memory kernel, whose tiles hold 256 tokens, needs no more).  A CTA that finds
    no tile leaves at once, but it holds an SM's shared memory while it looks, so a caller
    that knows the requests' token counts on the host passes them (``query_lengths``) and the
    grid is exactly the tiles there are.
    ``tensor_memory``: take the tcgen05 kernel (scores, probabilities and output in tensor
    memory; pages of at least 16 keys) or the ``mma.sync`` kernel; default: tcgen05 where it
    applies."""
    _need(q, torch.bfloat16, "q")
    _need(k_cache, torch.bfloat16, "k_cache")
    _need(out, torch.bfloat16, "out")
    if tensor_memory is None:
        tensor_memory = prefill_attention_tc_supports(head_dim, page_size)
    entry = lib().hx_prefill_attention_tc if tensor_memory else lib().hx_prefill_attention
    if query_lengths is not None:
        rows = PREFILL_TILE_ROWS_TC if tensor_memory else PREFILL_TILE_ROWS
        tile_bound = sum(-(-length // rows) for length in query_lengths
                         if length >= min_query_len)
        if tile_bound == 0:
            return
    _check(entry(
        q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), request_start.data_ptr(),
        request_context.data_ptr(), request_table_row.data_ptr(), block_tables.data_ptr(),
        block_tables.stride(0), out.data_ptr(), out.stride(0), requests, tile_bound, heads,
        kv_heads, head_dim, page_size, num_pages, float(scale), min_query_len, _ptr(status),
        _stream()))


def argmax(logits: torch.Tensor, tokens_out: torch.Tensor, status: Optional[torch.Tensor]) -> None:
    _need(logits, torch.float32, "logits")
    _need(tokens_out, torch.int32, "tokens_out")
    rows, vocab = logits.shape
    _check(lib().hx_argmax(logits.data_ptr(), logits.stride(0), rows, vocab, tokens_out.data_ptr(),
                           _ptr(status), _stream()))


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
           tokens_out: torch.Tensor, status: Optional[torch.Tensor]) -> None:
    _need(logits, torch.float32, "logits")
    _need(temperature, torch.float32, "temperature")
    _need(uniform, torch.float32, "uniform")
    _need(tokens_out, torch.int32, "tokens_out")
    rows, vocab = logits.shape
    _check(lib().hx_sample(logits.data_ptr(), logits.stride(0), rows, vocab, temperature.data_ptr(),
                           uniform.data_ptr(), tokens_out.data_ptr(), _ptr(status), _stream()))


def feed_tokens(token_ids: torch.Tensor, sampled: torch.Tensor, rows: torch.Tensor,
                count: int) -> None:
    """token_ids[i] = max(sampled[rows[i]], 0) for i < count: the tokens of a step that was
    prepared before the host had read what the step before it sampled."""
    _need(token_ids, torch.int32, "token_ids")
    _need(sampled, torch.int32, "sampled")
    _need(rows, torch.int32, "rows")
    _check(lib().hx_feed_tokens(token_ids.data_ptr(), sampled.data_ptr(), rows.data_ptr(), count,
                                sampled.shape[0], _stream()))


def launch_count() -> int:
    """Kernels this library has launched (or recorded into a graph) since it was loaded."""
    return int(lib().hx_launch_count())


def set_dependent_launch(enabled: bool) -> None:
    """Switch programmatic dependent launch of the kernels off (debugging) or on (default)."""
    lib().hx_set_dependent_launch(1 if enabled else 0)


def bounded_wait_check(polls: int, arrive: bool, status: torch.Tensor) -> bool:
    """Run the kernels' bounded mbarrier wait on a barrier of its own with a limit of ``polls``
    polls.  ``arrive`` False: nobody arrives, the wait runs out, the kernel sets
    FLAG_WAIT_TIMEOUT in ``status`` and returns.  Returns whether the wait succeeded."""
    succeeded = torch.full((1,), -1, dtype=torch.int32, device=status.device)
    _check(lib().hx_bounded_wait_check(int(polls), 1 if arrive else 0, _ptr(status),
                                       _ptr(succeeded), _stream()))
    return int(succeeded.item()) == 1
