"""Plain, slow implementation of the Llama-style MHA decoder, from the reference's formulas.

Whole sequences, no cache, one function per part, NumPy only, double accumulators
with a cast to float32 after every operation exactly where the reference's CPU
path casts.  It shares no code with the engine: it has its own safetensors reader
and its own checkpoint-layout conversion.  Paths cited are the reference
project's.

Checked once against the reference's own compiled CPU model
(``tests/golden/make_golden.py`` wrote ``tests/golden/*.json`` from
``helix_model_inspect``); ``tests/test_plain_reference.py`` replays that
comparison from the committed files.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np

F32 = np.float32
F64 = np.float64


# --------------------------------------------------------------------------- files

def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    """Every tensor of one safetensors file as float32 (bf16: bits << 16,
    tools/convert_hf_llama.py:528-532)."""
    with open(path, "rb") as source:
        (header_length,) = struct.unpack("<Q", source.read(8))
        header = json.loads(source.read(header_length).decode("utf-8"))
        payload = source.read()
    header.pop("__metadata__", None)
    tensors: Dict[str, np.ndarray] = {}
    for name, record in header.items():
        start, end = record["data_offsets"]
        raw = payload[start:end]
        shape = tuple(record["shape"])
        if record["dtype"] == "F32":
            value = np.frombuffer(raw, dtype="<f4").astype(F32)
        elif record["dtype"] == "F16":
            value = np.frombuffer(raw, dtype="<f2").astype(F32)
        elif record["dtype"] == "BF16":
            bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << np.uint32(16)
            value = bits.view(F32)
        else:
            raise ValueError(f"unsupported dtype {record['dtype']}")
        tensors[name] = value.reshape(shape)      # astype and the shift made fresh arrays
    return tensors


def read_model_folder(directory: str):
    with open(os.path.join(directory, "config.json"), "r", encoding="utf-8") as source:
        config = json.load(source)
    return config, read_safetensors(os.path.join(directory, "model.safetensors"))


# ------------------------------------------------------- checkpoint -> Helix layout

def rotary_output_permutation(heads: int, head_dim: int) -> np.ndarray:
    """Per head the new output order is ``[0, D/2, 1, D/2+1, ...]``
    (tools/convert_hf_llama.py:535-542): turns the checkpoint's half-split rotary
    convention into the adjacent-pair one."""
    half = head_dim // 2
    order: List[int] = []
    for head in range(heads):
        base = head * head_dim
        for frequency in range(half):
            order.extend((base + frequency, base + half + frequency))
    return np.asarray(order, dtype=np.intp)


def to_helix_layout(config: dict, source: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
    """``[out, in]`` checkpoint matrices -> the reference's ``[in, out]`` layout, with the
    rotary row permutation on Q and K only (tools/convert_hf_llama.py:400-510)."""
    heads = config["num_attention_heads"]
    head_dim = config["hidden_size"] // heads
    permutation = rotary_output_permutation(heads, head_dim)
    out: Dict[str, np.ndarray] = {"token_embedding": source["model.embed_tokens.weight"]}
    for layer in range(config["num_hidden_layers"]):
        prefix = f"model.layers.{layer}"
        out[f"layer.{layer}.attention_norm"] = source[f"{prefix}.input_layernorm.weight"]
        out[f"layer.{layer}.query"] = source[f"{prefix}.self_attn.q_proj.weight"][permutation].T
        out[f"layer.{layer}.key"] = source[f"{prefix}.self_attn.k_proj.weight"][permutation].T
        out[f"layer.{layer}.value"] = source[f"{prefix}.self_attn.v_proj.weight"].T
        out[f"layer.{layer}.attention_output"] = source[f"{prefix}.self_attn.o_proj.weight"].T
        out[f"layer.{layer}.ffn_norm"] = source[f"{prefix}.post_attention_layernorm.weight"]
        out[f"layer.{layer}.gate"] = source[f"{prefix}.mlp.gate_proj.weight"].T
        out[f"layer.{layer}.up"] = source[f"{prefix}.mlp.up_proj.weight"].T
        out[f"layer.{layer}.down"] = source[f"{prefix}.mlp.down_proj.weight"].T
    out["final_norm"] = source["model.norm.weight"]
    lm_source = "lm_head.weight"
    if lm_source not in source:
        # tied head: the embedding stands in (tools/convert_hf_llama.py:497-510)
        lm_source = "model.embed_tokens.weight"
    out["lm_head"] = source[lm_source].T
    return out


# ------------------------------------------------------------------------- the parts

def embedding_lookup(ids: Sequence[int], table: np.ndarray) -> np.ndarray:
    """``out[t, :] = table[id[t], :]`` (src/kernels/cpu/reference.cpp:426-455)."""
    ids = np.asarray(ids, dtype=np.int64)
    if ids.size and (ids.min() < 0 or ids.max() >= table.shape[0]):
        raise IndexError("token id outside the vocabulary")
    return table[ids].astype(F32)


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """``y = x / sqrt(mean(x^2) + eps) * w`` in double, one cast
    (src/kernels/cpu/reference.cpp:392-406).  eps is a float32 value in the reference."""
    wide = x.astype(F64)
    mean_square = (wide * wide).sum(axis=-1, keepdims=True) / x.shape[-1]
    inverse = 1.0 / np.sqrt(mean_square + F64(F32(eps)))
    return (wide * inverse * weight.astype(F64)).astype(F32)


def linear(x: np.ndarray, weight_in_out: np.ndarray) -> np.ndarray:
    """``y = x @ W`` with W ``[in, out]``, double accumulate, one cast
    (src/kernels/cpu/reference.cpp:349-358, 541-553)."""
    return (x.astype(F64) @ weight_in_out.astype(F64)).astype(F32)


def rope_table(tokens: int, head_dim: int, theta: float, offset: int = 0):
    """cos/sin ``[tokens, D/2]``: ``f_p = theta^(-2p/D)``, angle = position * f_p, in
    double, cast to float32 (src/model/llama_common.cpp:37-46).  theta is a float32 value."""
    pairs = head_dim // 2
    exponent = -2.0 * np.arange(pairs, dtype=F64) / F64(head_dim)
    frequency = np.power(F64(F32(theta)), exponent)
    positions = np.arange(offset, offset + tokens, dtype=F64)[:, None]
    angle = positions * frequency[None, :]
    return np.cos(angle).astype(F32), np.sin(angle).astype(F32)


def rope_adjacent(x: np.ndarray, cosine: np.ndarray, sine: np.ndarray) -> np.ndarray:
    """Rotate adjacent pairs ``(2p, 2p+1)`` of ``x [T, heads, D]`` in float32
    (src/kernels/cpu/reference.cpp:519-531)."""
    first = x[..., 0::2]
    second = x[..., 1::2]
    c = cosine[:, None, :]
    s = sine[:, None, :]
    out = np.empty_like(x)
    out[..., 0::2] = (first * c - second * s).astype(F32)
    out[..., 1::2] = (first * s + second * c).astype(F32)
    return out


def rope_half_split(x: np.ndarray, cosine: np.ndarray, sine: np.ndarray) -> np.ndarray:
    """The checkpoint's own convention: pair ``(p, p + D/2)``
    (tools/validate_hf_llama.py:373-544 uses it as the source-layout oracle)."""
    half = x.shape[-1] // 2
    first = x[..., :half]
    second = x[..., half:]
    c = cosine[:, None, :]
    s = sine[:, None, :]
    out = np.empty_like(x)
    out[..., :half] = (first * c - second * s).astype(F32)
    out[..., half:] = (first * s + second * c).astype(F32)
    return out


def softmax_rows(scores: np.ndarray) -> np.ndarray:
    """Row max in float32, exp and sum in double, one cast
    (src/kernels/cpu/reference.cpp:278-315).  Rows that hold NaN or only -inf become NaN."""
    maximum = scores.max(axis=-1, keepdims=True)
    with np.errstate(invalid="ignore"):
        shifted = (scores - maximum).astype(F32).astype(F64)
        numerator = np.exp(shifted)
        denominator = numerator.sum(axis=-1, keepdims=True)
        result = (numerator / denominator).astype(F32)
    bad = np.isnan(scores).any(axis=-1, keepdims=True) | np.isneginf(maximum)
    return np.where(bad, F32(np.nan), result)


def causal_attention(query: np.ndarray, key: np.ndarray, value: np.ndarray,
                     query_offset: int = 0, window: Optional[int] = None,
                     scale: Optional[float] = None) -> np.ndarray:
    """``softmax(q k^T / sqrt(D) + mask) v`` for ``query [A, Q, D]``, ``key/value [Akv, K, D]``.

    Mask: key ``k`` is hidden when ``k > query_offset + q``
    (src/attention/reference.cpp:154-176); scores in double times a double scale, cast to
    float32; probabilities times values accumulated in double (reference.cpp:181-224).
    ``Akv < A`` (grouped heads) and ``window`` (key also hidden when
    ``k <= query_offset + q - window``) are generalisations used by kernel tests only.
    """
    heads, queries, head_dim = query.shape
    kv_heads, keys, _ = key.shape
    group = heads // kv_heads
    if scale is None:
        scale = 1.0 / math.sqrt(float(head_dim))
    out = np.empty((heads, queries, value.shape[-1]), dtype=F32)
    q_pos = query_offset + np.arange(queries)[:, None]
    k_pos = np.arange(keys)[None, :]
    hidden = k_pos > q_pos
    if window is not None:
        hidden = hidden | (k_pos <= q_pos - window)
    for head in range(heads):
        kv = head // group
        scores = ((query[head].astype(F64) @ key[kv].astype(F64).T) * F64(scale)).astype(F32)
        scores = np.where(hidden, F32(-np.inf), scores)
        probabilities = softmax_rows(scores)
        out[head] = (probabilities.astype(F64) @ value[kv].astype(F64)).astype(F32)
    return out


def silu(x: np.ndarray) -> np.ndarray:
    """``x * sigmoid(x)`` with the branch-stable sigmoid, in double
    (src/kernels/cpu/reference.cpp:98-108)."""
    wide = x.astype(F64)
    with np.errstate(over="ignore"):
        positive = 1.0 / (1.0 + np.exp(-wide))
        exponential = np.exp(wide)
        negative = exponential / (1.0 + exponential)
    return (wide * np.where(x >= 0, positive, negative)).astype(F32)


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """``silu(gate) * up`` with the product in float32 (reference.cpp:415-418)."""
    return (silu(gate) * up).astype(F32)


# ------------------------------------------------------------------- the whole model

def round_bfloat16(x: np.ndarray) -> np.ndarray:
    """Round float32 values to the nearest bfloat16 (ties to even), kept as float32."""
    bits = np.ascontiguousarray(x, dtype=F32).view(np.uint32)
    rounded = (bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) \
        & np.uint32(0xFFFF0000)
    return rounded.view(F32)


def keep(x: np.ndarray) -> np.ndarray:
    return x


def attention_block(config: dict, weights: Dict[str, np.ndarray], layer: int,
                    normed: np.ndarray, offset: int = 0, store=keep) -> np.ndarray:
    """QKV projections, rotary encoding of Q and K, causal attention, output projection
    (src/model/cpu_llama.cpp:65-90).  ``store`` is applied wherever a bfloat16 engine keeps an
    activation in 16 bits; for the float32 model it is the identity."""
    tokens = normed.shape[0]
    heads = config["num_attention_heads"]
    head_dim = config["hidden_size"] // heads
    cosine, sine = rope_table(tokens, head_dim, config.get("rope_theta", 10000.0), offset)
    q = store(linear(normed, weights[f"layer.{layer}.query"])).reshape(tokens, heads, head_dim)
    k = store(linear(normed, weights[f"layer.{layer}.key"])).reshape(tokens, heads, head_dim)
    v = store(linear(normed, weights[f"layer.{layer}.value"])).reshape(tokens, heads, head_dim)
    q = store(rope_adjacent(q, cosine, sine)).transpose(1, 0, 2)
    k = store(rope_adjacent(k, cosine, sine)).transpose(1, 0, 2)
    v = v.transpose(1, 0, 2)
    context = store(causal_attention(q, k, v, query_offset=offset))
    merged = context.transpose(1, 0, 2).reshape(tokens, heads * head_dim)
    return linear(merged, weights[f"layer.{layer}.attention_output"])


def mlp_block(weights: Dict[str, np.ndarray], layer: int, normed: np.ndarray,
              store=keep) -> np.ndarray:
    """gate/up projections, SwiGLU, down projection (src/model/cpu_llama.cpp:94-97)."""
    gate = linear(normed, weights[f"layer.{layer}.gate"])
    up = linear(normed, weights[f"layer.{layer}.up"])
    return linear(store(swiglu(gate, up)), weights[f"layer.{layer}.down"])


def forward(config: dict, weights: Dict[str, np.ndarray], ids: Sequence[int],
            return_hidden: bool = False, precision: str = "float32"):
    """Logits ``[T, V]`` at every position of one whole sequence
    (src/model/cpu_llama.cpp:37-110).  ``weights`` are in Helix layout.

    ``precision="bfloat16"`` is the same model with the activations between the float32
    residual sums rounded to bfloat16 where a bfloat16 engine stores them (after each norm,
    after the Q/K/V projections and the rotation, after attention, after SwiGLU); all sums
    stay in double.  The reference has no such mode (README.md:693); it is here so that a
    bfloat16 engine can be held to a tolerance far below bfloat16's own rounding."""
    if len(ids) == 0:
        raise ValueError("token sequence must not be empty")
    if len(ids) > config["max_position_embeddings"]:
        raise ValueError("token sequence exceeds configured maximum")
    store = {"float32": keep, "bfloat16": round_bfloat16}[precision]
    eps = config.get("rms_norm_eps", 1.0e-6)
    hidden = embedding_lookup(ids, weights["token_embedding"])
    states = []
    for layer in range(config["num_hidden_layers"]):
        normed = store(rms_norm(hidden, weights[f"layer.{layer}.attention_norm"], eps))
        hidden = (hidden + attention_block(config, weights, layer, normed, store=store)).astype(F32)
        normed = store(rms_norm(hidden, weights[f"layer.{layer}.ffn_norm"], eps))
        hidden = (hidden + mlp_block(weights, layer, normed, store=store)).astype(F32)
        states.append(hidden)
    final = store(rms_norm(hidden, weights["final_norm"], eps))
    logits = linear(final, weights["lm_head"])
    if return_hidden:
        return logits, states
    return logits


def forward_source_layout(config: dict, source: Dict[str, np.ndarray],
                          ids: Sequence[int]) -> np.ndarray:
    """The same model straight from the checkpoint's layout: ``[out, in]`` matrices and
    half-split rotation (tools/validate_hf_llama.py:373-544).  Agreement with
    :func:`forward` checks the rotary row permutation."""
    eps = config.get("rms_norm_eps", 1.0e-6)
    heads = config["num_attention_heads"]
    head_dim = config["hidden_size"] // heads
    tokens = len(ids)
    cosine, sine = rope_table(tokens, head_dim, config.get("rope_theta", 10000.0))
    hidden = embedding_lookup(ids, source["model.embed_tokens.weight"])
    for layer in range(config["num_hidden_layers"]):
        prefix = f"model.layers.{layer}"
        normed = rms_norm(hidden, source[f"{prefix}.input_layernorm.weight"], eps)
        q = linear(normed, source[f"{prefix}.self_attn.q_proj.weight"].T)
        k = linear(normed, source[f"{prefix}.self_attn.k_proj.weight"].T)
        v = linear(normed, source[f"{prefix}.self_attn.v_proj.weight"].T)
        q = rope_half_split(q.reshape(tokens, heads, head_dim), cosine, sine).transpose(1, 0, 2)
        k = rope_half_split(k.reshape(tokens, heads, head_dim), cosine, sine).transpose(1, 0, 2)
        v = v.reshape(tokens, heads, head_dim).transpose(1, 0, 2)
        context = causal_attention(q, k, v).transpose(1, 0, 2).reshape(tokens, -1)
        hidden = (hidden + linear(context, source[f"{prefix}.self_attn.o_proj.weight"].T)).astype(F32)
        normed = rms_norm(hidden, source[f"{prefix}.post_attention_layernorm.weight"], eps)
        gate = linear(normed, source[f"{prefix}.mlp.gate_proj.weight"].T)
        up = linear(normed, source[f"{prefix}.mlp.up_proj.weight"].T)
        hidden = (hidden + linear(swiglu(gate, up), source[f"{prefix}.mlp.down_proj.weight"].T)).astype(F32)
    final = rms_norm(hidden, source["model.norm.weight"], eps)
    head = source.get("lm_head.weight", source["model.embed_tokens.weight"])
    return linear(final, head.T)


# ------------------------------------------------------------------------ generation

def select_greedy_token(logits_row: np.ndarray) -> int:
    """Lowest id among the maxima; non-finite logits are an error
    (src/model/cpu_generation.cpp:66-98)."""
    if not np.isfinite(logits_row).all():
        raise FloatingPointError("logits contain a non-finite value")
    return int(np.argmax(logits_row))


def greedy_generate(config: dict, weights: Dict[str, np.ndarray], prompt: Sequence[int],
                    max_new_tokens: int, eos: Optional[int] = None,
                    precision: str = "float32") -> List[int]:
    """Greedy continuation by full recomputation each step; stops at ``eos`` (emitted), at
    ``max_new_tokens`` or when the context is full (src/model/cpu_generation.cpp:137-167)."""
    tokens = list(prompt)
    generated: List[int] = []
    while len(generated) < max_new_tokens:
        token = select_greedy_token(forward(config, weights, tokens, precision=precision)[-1])
        generated.append(token)
        if eos is not None and token == eos:
            break
        if len(tokens) >= config["max_position_embeddings"]:
            break
        tokens.append(token)
    return generated


class PlainModel:
    """A model folder loaded for the plain implementation."""

    def __init__(self, directory: str, precision: str = "float32") -> None:
        self.config, self.source = read_model_folder(directory)
        self.weights = to_helix_layout(self.config, self.source)
        self.precision = precision

    def logits(self, ids: Sequence[int]) -> np.ndarray:
        return forward(self.config, self.weights, ids, precision=self.precision)

    def greedy(self, prompt: Sequence[int], max_new_tokens: int,
               eos: Optional[int] = None) -> List[int]:
        return greedy_generate(self.config, self.weights, prompt, max_new_tokens, eos,
                               precision=self.precision)
