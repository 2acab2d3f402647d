"""What the two command lines answer before any kernel runs: their options, the refusal of bad
values, and, on a machine without a GPU, the plain statement that there is no CPU path
(the reference's ``helix_generate`` prints the error and its usage and exits with 1,
examples/generate.cpp)."""
from __future__ import annotations

import os
import subprocess
import sys

import pytest
import torch

from conftest import ROOT
from tiny_configs import make_folder

GENERATE = os.path.join(ROOT, "bin", "helix_generate")
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def run(*command, stdin=""):
    return subprocess.run([sys.executable, *command], input=stdin, stdout=subprocess.PIPE,
                          stderr=subprocess.PIPE, text=True, timeout=300)


def test_generate_has_the_references_option_names():
    result = run(GENERATE, "--help")
    assert result.returncode == 0
    for option in ("--model", "--max-new-tokens", "--eos", "--temperature", "--seed", "--dtype",
                   "--random-weights"):
        assert option in result.stdout
    assert "TOKEN" in result.stdout


def test_generate_refuses_a_prompt_that_is_no_list_of_integers(tmp_path):
    result = run(GENERATE, "--model", str(tmp_path), "5", "seven")
    assert result.returncode == 2 and "invalid int value" in result.stderr
    result = run(GENERATE, "--model", str(tmp_path), "--max-new-tokens", "-1", "5")
    assert result.returncode == 2 and "nonnegative" in result.stderr


def test_trace_run_refuses_bad_sizes_before_it_loads_anything(tmp_path):
    common = ("--model", str(tmp_path), "--dtype", "float32", "--out", str(tmp_path / "out"))
    result = run(TRACE_RUN, *common, "--max-tokens", "0")
    assert result.returncode == 2 and "--max-tokens must be positive" in result.stderr
    result = run(TRACE_RUN, *common, "--max-tokens", "64", "--page-size", "24")
    assert result.returncode == 2 and "--page-size must divide 64" in result.stderr
    result = run(TRACE_RUN, "--model", str(tmp_path), "--dtype", "float16", "--out", "x",
                 "--max-tokens", "64")
    assert result.returncode == 2 and "invalid choice" in result.stderr


@pytest.mark.skipif(torch.cuda.is_available(), reason="needs a machine without a GPU")
def test_without_a_gpu_both_say_that_there_is_no_cpu_path(model_root):
    folder = make_folder(model_root, "A", storage_dtype="float32")
    result = run(GENERATE, "--model", folder, "--dtype", "float32", "5", "17", "3")
    assert result.returncode == 1
    assert "no CPU path" in result.stderr and "usage: helix_generate" in result.stderr
    assert result.stdout == ""
    result = run(TRACE_RUN, "--model", folder, "--dtype", "float32", "--out",
                 os.path.join(model_root, "logits"), "--max-tokens", "64",
                 stdin='{"step": 0, "entries": [{"id": "a", "tokens": [1, 2], "want": [1]}]}\n')
    assert result.returncode != 0 and "no CPU path" in result.stderr
    assert "done" not in result.stdout
