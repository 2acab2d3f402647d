"""Shared fixtures.  Tests that need a GPU carry ``@pytest.mark.gpu``; everything else runs
on a machine without one."""
from __future__ import annotations

import os
import sys

import numpy as np
import pytest

TESTS = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(TESTS)
for path in (ROOT, TESTS):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs an NVIDIA B200 (run with -m gpu)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_root(tmp_path_factory):
    """A temporary folder in which tests make their model folders; never committed."""
    return str(tmp_path_factory.mktemp("models"))


@pytest.fixture(scope="session")
def folders(model_root):
    """``folders(name, storage_dtype, sharp)`` -> path of that tiny model folder."""
    from tiny_configs import make_folder

    def get(name: str, storage_dtype: str = "float32", sharp: bool = True) -> str:
        return make_folder(model_root, name, storage_dtype=storage_dtype, sharp=sharp)
    return get


@pytest.fixture(scope="session")
def plain_models(folders):
    """``plain_models(name, dtype, sharp)`` -> the plain implementation of that folder, with
    activations rounded where a bfloat16 engine stores them when ``dtype`` is bfloat16."""
    import plain_llama
    cache = {}

    def get(name: str, storage_dtype: str = "float32", sharp: bool = True):
        key = (name, storage_dtype, sharp)
        if key not in cache:
            cache[key] = plain_llama.PlainModel(folders(name, storage_dtype, sharp),
                                                precision=storage_dtype)
        return cache[key]
    return get


def random_tokens(vocab: int, count: int, seed: int):
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, vocab, size=count)]
