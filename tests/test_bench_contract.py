"""What ``bench.py`` answers without a GPU: more than one GPU is refused with exit code 2, the
reference arm says why it is unavailable, other shapes go with the serving and profiling modes
only; and the rule by which the attention part widens a head."""
from __future__ import annotations

import json
import os
import subprocess
import sys

from conftest import ROOT

BENCH = os.path.join(ROOT, "bench.py")


def run_bench(*arguments):
    return subprocess.run([sys.executable, BENCH, *arguments], stdout=subprocess.PIPE,
                          stderr=subprocess.PIPE, text=True, timeout=300)


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2():
    result = run_bench("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert result.returncode == 2
    lines = [line for line in result.stdout.splitlines() if line.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_prints_why_it_is_unavailable():
    result = run_bench("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert result.returncode == 0
    record = json.loads(result.stdout.strip().splitlines()[-1])
    assert record["impl"] == "reference" and len(record["unavailable"]) > 20


def test_other_shapes_belong_to_the_serving_and_profiling_modes():
    result = run_bench("--shape", "llama-2-13b")
    assert result.returncode == 2 and "--serving" in result.stdout


def test_benchmark_shapes_are_valid_configurations():
    sys.path.insert(0, ROOT)
    import bench
    from helix_runtime_b200 import LlamaConfig

    assert set(bench.WORKLOADS) == set(bench.SHAPES)
    for name, shape in bench.SHAPES.items():
        config = LlamaConfig(**shape)
        assert config.num_attention_heads == config.num_key_value_heads, name
        work = bench.WORKLOADS[name]
        low, high = work["prompt_range"]
        assert 0 < low < high <= config.max_position_embeddings
        assert work["shared_prefix"] + work["new_tokens"] < config.max_position_embeddings


def test_heads_are_held_in_rows_the_tensor_core_kernels_tile():
    from helix_runtime_b200.parts.attention import row_width

    # steps of 16 up to 128, of 32 up to 256, as it is beyond that
    assert [row_width(d) for d in (2, 16, 24, 100, 112, 128)] == [16, 16, 32, 112, 112, 128]
    assert [row_width(d) for d in (130, 144, 160, 250, 256, 258, 512)] == \
        [160, 160, 160, 256, 256, 258, 512]
