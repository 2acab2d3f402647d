"""The engine for C and C++ callers (``include/helix_b200/engine.h``).

``tests/cpp/generate_tiny.cpp`` is a C++ program that links the interface library, creates an
engine from a model path, submits, cancels, runs until done and prints what the command line
tool prints.  On a GPU it must generate, from the model file that the reference's own tools
packed, the tokens that the reference's CPU model generated (``tests/golden``).  Without a
GPU the same program must fail with the engine's own message, which shows that the embedded
interpreter, the package and the error path work.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys

import pytest

from conftest import ROOT

GOLDEN = os.path.join(ROOT, "tests", "golden")
SOURCE = os.path.join(ROOT, "tests", "cpp", "generate_tiny.cpp")


@pytest.fixture(scope="module")
def program(tmp_path_factory):
    from helix_runtime_b200.csrc import build
    library = build.build_engine_api()
    folder = os.path.dirname(library)
    binary = str(tmp_path_factory.mktemp("cpp") / "generate_tiny")
    subprocess.run([build.find_cxx(), "-std=c++17", "-Wall", "-Wextra", "-Werror", SOURCE,
                    f"-I{os.path.join(ROOT, 'include')}", f"-L{folder}", "-lhelix_b200_engine",
                    f"-Wl,-rpath,{folder}", "-o", binary], check=True)
    return binary


def run(program, *arguments):
    environment = dict(os.environ, HELIX_B200_PYTHON=sys.executable)
    environment.pop("PYTHONPATH", None)            # the library finds the package by itself
    return subprocess.run([program, *map(str, arguments)], capture_output=True, text=True,
                          env=environment, cwd="/", timeout=600)


def test_header_is_plain_c_too(tmp_path):
    source = tmp_path / "only_c.c"
    source.write_text('#include "helix_b200/engine.h"\n'
                      "int main(void) { hxe_config c = {0}; return c.page_size; }\n")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-c", str(source),
                    f"-I{os.path.join(ROOT, 'include')}", "-o", str(tmp_path / "only_c.o")],
                   check=True)


def test_without_a_gpu_the_cpp_caller_gets_the_engines_message(program):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the other test runs the program")
    result = run(program, os.path.join(GOLDEN, "tiny_A.helix"), "float32", 4, 1, 2, 3)
    assert result.returncode == 1
    assert "generate_tiny: RuntimeError: no CUDA device is available" in result.stderr
    result = run(program, "/nonexistent/model", "float32", 4, 1, 2, 3)
    assert result.returncode == 1 and "generate_tiny:" in result.stderr


@pytest.mark.gpu
def test_cpp_caller_generates_the_references_tokens(program):
    with open(os.path.join(GOLDEN, "tiny_A.json"), "r", encoding="utf-8") as source:
        golden = json.load(source)
    greedy = golden["greedy"]
    prompt = golden["tokens"][:greedy["prompt_length"]]
    result = run(program, os.path.join(GOLDEN, "tiny_A.helix"), "float32", len(greedy["tokens"]),
                 *prompt)
    assert result.returncode == 0, result.stderr
    lines = result.stdout.strip().splitlines()
    assert [int(t) for t in lines[0].split(":", 1)[1].split()] == greedy["tokens"]
    assert lines[1] == "stop_reason: max_new_tokens"
    assert lines[2] == f"cached_token_count: {len(prompt) + len(greedy['tokens']) - 1}"
    facts = dict(item.split("=") for item in lines[3].split())
    assert facts["finished"] == "1" and facts["cancelled"] == "1" and facts["state"] == "4"
    assert facts["free_pages"] == facts["pages"]            # everything was given back
    # a prompt token outside the vocabulary is the engine's refusal, as an exception's text
    bad = run(program, os.path.join(GOLDEN, "tiny_A.helix"), "float32", 3, 1, 99999)
    assert bad.returncode == 1 and "outside the vocabulary" in bad.stderr
