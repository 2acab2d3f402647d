"""``bin/trace_run`` as a user runs it: a subprocess fed JSON lines, logits read from files.

The same requests are replayed whole, with the last 32 tokens decoded one by one, in portions
of changing size, and mixed with other requests in a pool so small that pages are used again,
in float32 and in bfloat16, and every logit row is compared with the plain implementation.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import pytest

import traces
from conftest import ROOT, random_tokens
from engine_harness import assert_close, tolerance
from tiny_configs import tiny_config

pytestmark = pytest.mark.gpu

TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")
LENGTHS = {"A": (33, 60, 97), "B": (40, 100, 160), "C": (50, 130, 260)}


def requests_for(name):
    vocab = tiny_config(name).vocab_size
    return {f"q{index}": random_tokens(vocab, length, seed=31 * ord(name) + index)
            for index, length in enumerate(LENGTHS[name])}


def run_trace(folder, dtype, steps, out_dir, max_tokens):
    process = subprocess.Popen(
        [sys.executable, TRACE_RUN, "--model", folder, "--dtype", dtype, "--out", out_dir,
         "--max-tokens", str(max_tokens)],
        stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, cwd=ROOT)
    try:
        for step in steps:
            process.stdin.write(json.dumps(step) + "\n")
            process.stdin.flush()
            line = process.stdout.readline().strip()
            assert line == f"done {step['step']}", f"expected 'done {step['step']}', got {line!r}"
        process.stdin.close()
        assert process.wait(timeout=120) == 0
    finally:
        if process.poll() is None:
            process.kill()


def check(folder, plain, dtype, steps, tmp_path, what, name=""):
    out_dir = str(tmp_path / what.replace(" ", "_"))
    run_trace(folder, dtype, steps, out_dir, traces.live_token_need(steps, 64))
    vocab = plain.config["vocab_size"]
    expected = {}
    positions = {}
    for step in steps:
        rows = traces.labels(step, positions)
        path = os.path.join(out_dir, f"{step['step']}.f32")
        if not rows:
            assert not os.path.exists(path)
            continue
        data = np.fromfile(path, dtype="<f4").reshape(len(rows), vocab)
        want = []
        for request, position in rows:
            if request not in expected:
                expected[request] = plain.logits(what_tokens[request])
            want.append(expected[request][position])
        assert_close(data, np.stack(want), f"{what}, step {step['step']}",
                     **tolerance(dtype, name))


what_tokens = {}


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"),
                                        ("A", "bfloat16"), ("B", "bfloat16"),
                                        ("C", "bfloat16")])
def test_replay_every_way_of_cutting(name, dtype, folders, plain_models, tmp_path):
    folder = folders(name, dtype)
    plain = plain_models(name, dtype)
    requests = requests_for(name)
    what_tokens.clear()
    what_tokens.update(requests)
    check(folder, plain, dtype, traces.whole(requests), tmp_path, "whole", name)
    check(folder, plain, dtype, traces.tail_decoded(requests, 32), tmp_path, "tail decoded", name)
    check(folder, plain, dtype, traces.chunked(requests), tmp_path, "portions", name)
    doubled = dict(requests)
    doubled.update({f"again_{key}": value for key, value in requests.items()})
    what_tokens.update(doubled)
    check(folder, plain, dtype, traces.mixed(doubled, max_live=4, seed=3), tmp_path, "mixed",
          name)


def test_steps_that_want_nothing_write_no_file_and_requests_may_pause(folders, plain_models, tmp_path):
    folder = folders("A", "float32")
    plain = plain_models("A", "float32")
    a = random_tokens(256, 20, seed=1)
    b = random_tokens(256, 9, seed=2)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:10], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": b, "want": [8]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": a[10:], "want": [0, 9]}], "end": ["a"]},
    ]
    out_dir = str(tmp_path / "pause")
    run_trace(folder, "float32", steps, out_dir, 128)
    assert sorted(os.listdir(out_dir)) == ["1.f32", "2.f32"]
    got = np.fromfile(os.path.join(out_dir, "2.f32"), dtype="<f4").reshape(2, 256)
    assert_close(got, plain.logits(a)[[10, 19]], "paused request", **tolerance("float32"))
    got = np.fromfile(os.path.join(out_dir, "1.f32"), dtype="<f4").reshape(1, 256)
    assert_close(got, plain.logits(b)[[8]], "other request", **tolerance("float32"))
