"""The tiny configurations the tests use, and how their model folders are made.

A and B differ in every size and option: layers 2/3, hidden 64/120, heads 4/5, head size
16/24, intermediate 176/320 (neither a multiple of 64), vocabulary 256/384, rope theta
1e4/5e5, eps 1e-5/1e-6, positions 128/256, page size 8/16.  Their head sizes keep them on
the general kernels.  C is still small but has the shapes the fast kernels are built for
(head size 64, pages of 16, an intermediate size that is a multiple of 128, prompts of
hundreds of tokens fit), so that the tcgen05 products with tiled weights, the tcgen05 prompt
attention and the streaming decode attention are also checked through the whole model.
Norm weights are drawn around one (not exactly one) so that a norm that forgot its weight
would show.
"""
from __future__ import annotations

import os

from helix_runtime_b200 import LlamaConfig, write_random_model

TINY_A = dict(vocab_size=256, hidden_size=64, intermediate_size=176, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=4, head_dim=16,
              max_position_embeddings=128, rms_norm_eps=1e-5, rope_theta=10000.0)
TINY_B = dict(vocab_size=384, hidden_size=120, intermediate_size=320, num_hidden_layers=3,
              num_attention_heads=5, num_key_value_heads=5, head_dim=24,
              max_position_embeddings=256, rms_norm_eps=1e-6, rope_theta=500000.0)
TINY_C = dict(vocab_size=512, hidden_size=256, intermediate_size=384, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=4, head_dim=64,
              max_position_embeddings=512, rms_norm_eps=1e-5, rope_theta=10000.0)
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C}
PAGE_SIZE = {"A": 8, "B": 16, "C": 16}
SEED = {"A": 0, "B": 1, "C": 2}


def tiny_config(name: str) -> LlamaConfig:
    return LlamaConfig(**TINY[name])


# Attention of a tiny N(0, 0.02) model is almost uniform, which would hide a key that is
# missing or misplaced.  The sharp variant multiplies the query and key projections by a gain
# chosen so that attention scores have a spread (standard deviation) of about 1.5 whatever the
# width: score spread = gain^2 * std^2 * hidden, so single keys matter but the softmax is
# not one-hot.
SCORE_SPREAD = 1.5


def sharp_gains(name: str, std: float = 0.02):
    hidden = TINY[name]["hidden_size"]
    gain = (SCORE_SPREAD / (std * std * hidden)) ** 0.5
    return {"q_proj": gain, "k_proj": gain}


def make_folder(directory: str, name: str, storage_dtype: str = "float32",
                scale_std: float = 0.1, std: float = 0.02, sharp: bool = False) -> str:
    """Write the model folder of tiny configuration ``name`` under ``directory``."""
    path = os.path.join(directory, f"tiny_{name}_{storage_dtype}" + ("_sharp" if sharp else ""))
    if not os.path.exists(os.path.join(path, "model.safetensors")):
        write_random_model(path, tiny_config(name), SEED[name], std=std, scale_std=scale_std,
                           storage_dtype=storage_dtype,
                           gains=sharp_gains(name, std) if sharp else None)
    return path
