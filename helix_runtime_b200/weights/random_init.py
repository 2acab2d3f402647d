"""Seeded random weights: write a model folder from a configuration and a seed.

The reference has only ``Tensor::random_uniform`` (src/tensor/tensor.cpp:169-191)
and hand-made patterns in its tests; a seeded N(0, std) fill with norm weights
of one is this engine's own.  The folder has the checkpoint layout the
reference's converter reads (tools/convert_hf_llama.py:400-510): Hugging Face
tensor names, ``[out, in]`` matrices, half-split rotary row order.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Mapping, Optional, Sequence

import torch

from .loader import TensorRequest
from .safetensors_io import write_safetensors


def random_tensors(requests: Sequence[TensorRequest], seed: int, std: float = 0.02,
                   scale_std: float = 0.0,
                   storage_dtype: torch.dtype = torch.bfloat16,
                   gains: Optional[Mapping[str, float]] = None) -> Dict[str, torch.Tensor]:
    """Draw every requested tensor from one generator, in request order.

    Matrices and tables of embeddings are N(0, std) in ``storage_dtype``; scale
    vectors (norm weights) are ``1 + N(0, scale_std)`` stored in float32.  ``gains``
    multiplies every matrix whose name contains a key by that key's factor (tests
    sharpen the attention of tiny models this way, so that a misplaced key shows).
    """
    generator = torch.Generator(device="cpu")
    generator.manual_seed(int(seed))
    tensors: Dict[str, torch.Tensor] = {}
    for request in requests:
        if request.role == "scale":
            value = torch.ones(request.shape, dtype=torch.float32)
            if scale_std > 0.0:
                value = value + scale_std * torch.randn(request.shape, generator=generator,
                                                        dtype=torch.float32)
            tensors[request.name] = value
        elif request.role == "table":
            raise ValueError("integer tables have no random initialisation")
        else:
            value = torch.randn(request.shape, generator=generator, dtype=torch.float32) * std
            for key, factor in (gains or {}).items():
                if key in request.name:
                    value = value * factor
            tensors[request.name] = value.to(storage_dtype)
    return tensors


def write_model_folder(directory: str, config_document: dict, tensors: Dict[str, torch.Tensor]) -> None:
    os.makedirs(directory, exist_ok=True)
    with open(os.path.join(directory, "config.json"), "w", encoding="utf-8") as output:
        json.dump(config_document, output, indent=2)
        output.write("\n")
    write_safetensors(os.path.join(directory, "model.safetensors"), tensors)
