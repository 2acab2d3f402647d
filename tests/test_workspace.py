"""The step's named scratch buffers: same name, same memory; a buffer that has to be replaced
stays alive, because CUDA graphs recorded earlier still point at it."""
from __future__ import annotations

import torch

from helix_runtime_b200.parts.base import Workspace

CPU = torch.device("cpu")


def test_a_name_gives_the_same_memory_again():
    workspace = Workspace(CPU)
    first = workspace.get("x", (4, 8), torch.float32)
    assert workspace.get("x", (4, 8), torch.float32) is first
    zeros = workspace.accumulator("sum", (3,), torch.int32)
    assert zeros.eq(0).all() and workspace.accumulator("sum", (3,), torch.int32) is zeros
    flat = workspace.at_least("scratch", 100, torch.float32)
    assert workspace.at_least("scratch", 60, torch.float32) is flat


def test_a_replaced_buffer_is_kept_and_growth_at_least_doubles():
    workspace = Workspace(CPU)
    small = workspace.at_least("scratch", 100, torch.float32)
    address = small.data_ptr()
    grown = workspace.at_least("scratch", 101, torch.float32)
    assert grown is not small and grown.numel() >= 200
    assert any(kept is small for kept in workspace._retired) and small.data_ptr() == address
    shaped = workspace.get("x", (4, 8), torch.float32)
    reshaped = workspace.get("x", (8, 8), torch.float32)
    assert reshaped is not shaped and any(kept is shaped for kept in workspace._retired)
    assert workspace.bytes() == 4 * (100 + grown.numel() + 32 + 64)


def test_clearing_accumulators_reaches_the_replaced_ones_too():
    workspace = Workspace(CPU)
    old = workspace.accumulator("sum", (4,))
    old.fill_(3.0)
    new = workspace.accumulator("sum", (8,))
    new.fill_(5.0)
    workspace.clear_accumulators()
    assert old.eq(0).all() and new.eq(0).all()
