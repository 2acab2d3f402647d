#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Llama-2-7B shape, bfloat16, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]

Prints ONE JSON line.  A step is one decode step of the batch.  Every decode number is taken
on the path generation uses: ``Engine.submit`` and ``Engine.run_iteration`` (the scheduler,
the step function, CUDA graphs of the decode step, the next step queued on the device before
this one's tokens are read); there is no second decode driver.

* ``value``: decoded tokens per second at the default batch of 8, timed ON THE DEVICE with
  CUDA events around K iterations.  The loop of K steps is repeated with fresh requests until
  at least a second has been timed; ``ms_per_step`` is the median of the repeats, with the
  fastest and slowest beside it.
* ``e2e``: the same loop timed by the host's clock around the public calls, with a device
  synchronisation on both sides: every step copies its inputs from pinned host memory to the
  device and reads the sampled tokens back.
* The workload is the reference's: 512-token prompts, 256 generated tokens, so contexts from
  512 to 767, 640 on average.  K steps cannot cover that range for every K, so each repeat is
  placed in its middle: its requests bring prompts of ``640 - W - K/2`` tokens, and the timed
  steps run at contexts around 640 (``config.timed_prompt_len``, ``config.timed_context_mean``).
* ``prefill``: one 2,048-token prompt in one step.  ``roofline``: the bytes the decode step
  has to read (every weight once, the cache of the live requests) over its time, against the
  measured copy bandwidth.  ``points``: decoding at batch 1 and 64, with their fractions.

Weights are random, N(0, 0.02) from a fixed seed, made on the device; prompts are seeded
uniform token ids.  Every step streams more weight bytes than the L2 cache holds, so no L2
flush is needed between timed iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Llama-2-7B shape (the benchmark configuration)
SHAPE = dict(vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
             num_attention_heads=32, num_key_value_heads=32, head_dim=128,
             max_position_embeddings=4096, rms_norm_eps=1e-5, rope_theta=10000.0)
# the other two shapes of the reference's benchmark configurations (--shape, serving mode)
SHAPES = {
    "llama-2-7b": SHAPE,
    "openllama-3b": dict(vocab_size=32000, hidden_size=3200, intermediate_size=8640,
                         num_hidden_layers=26, num_attention_heads=32, num_key_value_heads=32,
                         head_dim=100, max_position_embeddings=2048, rms_norm_eps=1e-6,
                         rope_theta=10000.0),
    "llama-2-13b": dict(vocab_size=32000, hidden_size=5120, intermediate_size=13824,
                        num_hidden_layers=40, num_attention_heads=40, num_key_value_heads=40,
                        head_dim=128, max_position_embeddings=4096, rms_norm_eps=1e-5,
                        rope_theta=10000.0),
}
# serving workloads of those configurations: requests, prompt lengths, new tokens, prompt
# portion, length of the prefix all prompts share (0: none)
WORKLOADS = {
    "llama-2-7b": dict(prompt_range=(128, 2048), new_tokens=256, chunk=512, shared_prefix=0),
    "openllama-3b": dict(prompt_range=(64, 1024), new_tokens=128, chunk=512, shared_prefix=256),
    "llama-2-13b": dict(prompt_range=(128, 2048), new_tokens=256, chunk=512, shared_prefix=0),
}
PROMPT_LEN = 512             # the workload: prompts of 512 tokens, 256 generated
GENERATED = 256
MIN_TIMED_SECONDS = 1.0
PAGE_SIZE = 16
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path, "r", encoding="utf-8") as source:
            data = json.load(source)
        peaks = dict(FALLBACK_PEAKS)
        for key in peaks:
            if isinstance(data.get(key), (int, float)):
                peaks[key] = float(data[key])
        peaks["source"] = "measured"
        return peaks
    except (OSError, ValueError):
        return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, path: str) -> None:
        self.path = path
        self.process = None

    def start(self) -> None:
        try:
            self.handle = open(self.path, "w")
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=self.handle, stderr=subprocess.DEVNULL)
        except OSError:
            self.process = None

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        self.handle.close()
        clocks, maxima, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        with open(self.path, "r") as source:
            for line in source:
                fields = [f.strip() for f in line.split(",")]
                if len(fields) < 8:
                    continue
                try:
                    clocks.append(float(fields[0]))
                    maxima.append(float(fields[1]))
                except ValueError:
                    continue
                for name, value in zip(names, fields[4:8]):
                    if value.lower().startswith("active"):
                        reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None,
                "samples": len(clocks), "reasons": sorted(reasons)}


def reference_arm() -> int:
    print(json.dumps({
        "impl": "reference",
        "unavailable": "pip install of the reference fails: it is a C++/CMake project with no "
                       "setup.py or pyproject.toml; its CUDA path has never run on a GPU and its "
                       "validated path is single-threaded FP32 on the CPU, which cannot run the "
                       "Llama-2-7B benchmark configuration in minutes"}))
    return 0


def serving_workload(options, model, config, rng) -> int:
    """Continuous batching through the Python entry point, not part of the contract line:
    ``--serving N`` requests of the workload that goes with ``--shape`` (Llama-2-7B and 13B
    shapes: prompts of 128 to 2,048 tokens, 256 new tokens each, prompt portions of 512 tokens
    interleaved with decoding; OpenLLaMA-3B shape: prompts of 64 to 1,024 tokens that share
    their first 256, 128 new tokens each, prefix pages shared), the cache pool sized from the
    memory that is free after the weights.  Prints one JSON line."""
    import torch

    from helix_runtime_b200 import Engine, EngineConfig

    requests = options.serving
    work = WORKLOADS[options.shape]
    low, high = work["prompt_range"]
    high = min(high, config.max_position_embeddings - work["new_tokens"])
    shared = [int(t) for t in rng.integers(0, config.vocab_size, work["shared_prefix"])]
    prompts = []
    for _ in range(requests):
        length = max(int(rng.integers(low, high + 1)), len(shared) + 1)
        prompts.append(shared + [int(t) for t in rng.integers(0, config.vocab_size,
                                                              length - len(shared))])
    submitted = sum(len(prompt) for prompt in prompts)
    engine = Engine(model, EngineConfig(page_size=PAGE_SIZE, max_running_requests=min(requests, 64),
                                        max_tokens_per_iteration=PREFILL_TOKENS,
                                        max_prefill_chunk=work["chunk"],
                                        cache_memory_fraction=options.cache_fraction,
                                        prefix_cache_entries=8 if shared else 0))
    torch.cuda.synchronize()
    begin = time.perf_counter()
    iterations = 0
    if shared:
        # the first request brings the shared beginning into the cache (its pages are kept
        # when its prompt is done); the others arrive after that and find them
        first = engine.submit(prompts[0], max_new_tokens=work["new_tokens"])
        while engine.request(first).state.value in ("waiting", "prefill"):
            engine.run_iteration()
            iterations += 1
        prompts = prompts[1:]
    for prompt in prompts:
        engine.submit(prompt, max_new_tokens=work["new_tokens"])
    iterations += engine.run_until_done()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - begin
    metrics, stats = engine.metrics(), engine.stats()
    reused = stats["prefix"]["reused_tokens"] if stats["prefix"] else 0      # found in the cache
    print(json.dumps({
        "metric": f"serving: generated tokens/s over the whole run ({options.shape} shape, bf16)",
        "value": round(metrics.generated_tokens / seconds, 1), "unit": "tokens/s",
        "processed_tokens_per_s": round((metrics.generated_tokens + metrics.prompt_tokens_processed
                                         - reused) / seconds, 1),
        "requests": requests, "seconds": round(seconds, 3), "iterations": iterations,
        "prompt_tokens_submitted": submitted,
        "prefix": stats["prefix"],
        "prompt_tokens": metrics.prompt_tokens_processed,
        "generated_tokens": metrics.generated_tokens,
        "shared_prefix": len(shared),
        "time_to_first_token_p50_p95_s": [round(metrics.time_to_first_token.p50_seconds, 3),
                                          round(metrics.time_to_first_token.p95_seconds, 3)],
        "inter_token_p50_p95_ms": [round(metrics.inter_token_latency.p50_seconds * 1e3, 2),
                                   round(metrics.inter_token_latency.p95_seconds * 1e3, 2)],
        "cache_pages": engine.cache.groups[0].pool.num_pages,
        "steps_queued_ahead": stats["steps_queued_ahead"],
        "graphs_recorded": engine.graphs.captures, "layers": config.num_hidden_layers,
        "impl": "ours"}))
    return 0


def profile_region(options, model, config, fresh, rng) -> int:
    """One eager step (no CUDA graph) inside a profiler range: a decode step of ``--batch``
    requests at context ``--prompt-len``, or a prefill step of ``--prompt-len`` tokens."""
    import torch

    from helix_runtime_b200.engine.step import StepEntry

    length = options.prompt_len
    batch = options.batch if options.profile == "decode" else 1
    cache, step, sampler = fresh(batch, length + 8, max(length, batch, PREFILL_TOKENS))
    prompts = [[int(t) for t in rng.integers(0, config.vocab_size, length)] for _ in range(batch)]
    for index in range(batch):
        cache.admit(index)
    if options.profile == "prefill":
        step.run([StepEntry(0, prompts[0], [length - 1])])      # warm-up (sizes workspaces)
        cache.release(0)
        cache.admit(0)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        step.run([StepEntry(0, prompts[0], [length - 1])])
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        return 0
    per_step = max(1, PREFILL_TOKENS // length)
    for begin in range(0, batch, per_step):
        step.run([StepEntry(index, prompts[index], [length - 1])
                  for index in range(begin, min(begin + per_step, batch))])
    decode = [StepEntry(index, [1 + index], [0]) for index in range(batch)]
    for _ in range(2):
        sampler.launch(step.run(decode), True, step.status)
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    sampler.launch(step.run(decode), True, step.status)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    return 0


def timeline_region(options, model, config, fresh, rng) -> int:
    """The kernels of the step as they run in place (``--timeline decode``: four decode steps of
    ``--batch`` requests through the engine, CUDA graphs and early launches as in serving;
    ``--timeline prefill``: one step of ``--prompt-len`` tokens; ``--timeline mixed``: one step
    of four 512-token prompt portions at contexts 1,536 to 0 beside ``--batch`` decode tokens
    at a context of ``--prompt-len``), recorded with CUPTI through
    ``torch.profiler``: launches, mean duration and mean EXCLUSIVE time per kernel (the part of
    a kernel after every earlier kernel has ended: a kernel that was let in early spends the
    rest of its duration waiting for its predecessor).  Unlike an ncu capture nothing is
    serialised or replayed, so the times add up to the step."""
    import collections

    import torch
    from torch.profiler import ProfilerActivity, profile

    from helix_runtime_b200 import Engine, EngineConfig
    from helix_runtime_b200.engine.step import StepEntry

    length, batch = options.prompt_len, options.batch
    if options.timeline == "prefill":
        cache, step, _ = fresh(1, length + 8, length)
        prompt = [int(t) for t in rng.integers(0, config.vocab_size, length)]

        def run():
            cache.admit(0)
            step.run([StepEntry(0, prompt, [length - 1])], check_status=False)
            cache.release(0)
        steps = 1
    elif options.timeline == "mixed":
        # a serving step: four prompt portions of 512 tokens that go on from 1,536, 1,024, 512
        # and 0 cached tokens (the request admitted first is furthest along), beside --batch
        # decode tokens at a context of --prompt-len
        contexts = (1536, 1024, 512, 0)
        cache, step, _ = fresh(batch + len(contexts), max(length, max(contexts) + 512) + 8,
                               PREFILL_TOKENS + batch)
        draw = lambda count: [int(t) for t in rng.integers(0, config.vocab_size, count)]
        for request in range(batch + len(contexts)):
            cache.admit(request)
        for request in range(batch):                       # bring the decode requests to length
            step.run([StepEntry(request, draw(length), [])], check_status=False)
        for index, context in enumerate(contexts):
            if context:
                step.run([StepEntry(batch + index, draw(context), [])], check_status=False)

        def run():
            # running requests first, then the prompts: the order the scheduler gives a step
            entries = [StepEntry(request, draw(1), [0]) for request in range(batch)]
            entries += [StepEntry(batch + index, draw(512), [511]) for index in range(len(contexts))]
            ctx, want_rows, n_want, _ = step.prepare(entries)
            model.forward(ctx, cache, want_rows, n_want)
            torch.cuda.synchronize()
            step.fail(entries)      # nothing is published: the next run repeats the same step
        steps = 1
    else:
        # the first requests decode while the prompts of the last are still being fed: every
        # request gets tokens enough to be decoding still when the recorded steps are over
        feeding = -(-batch * length // PREFILL_TOKENS) + batch
        budget = min(feeding + 48, config.max_position_embeddings - length)
        if budget < feeding + 17:
            raise SystemExit(f"bench.py: {batch} prompts of {length} tokens leave no room to "
                             f"decode within {config.max_position_embeddings} positions")
        engine = Engine(model, EngineConfig(
            page_size=PAGE_SIZE, max_running_requests=batch,
            max_tokens_per_iteration=PREFILL_TOKENS,
            num_pages=batch * -(-(length + budget) // PAGE_SIZE) + 8))
        for _ in range(batch):
            engine.submit([int(t) for t in rng.integers(0, config.vocab_size, length)],
                          max_new_tokens=budget)
        for _ in range(4 * feeding + 16):
            if all(engine.request(r).state.value == "decoding" for r in range(batch)):
                break
            engine.run_iteration()
        else:
            raise SystemExit("bench.py: the requests did not all reach decoding")
        run, steps = engine.run_iteration, 4
    for _ in range(12 if options.timeline == "decode" else 3):
        run()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as recorded:
        for _ in range(steps):
            run()
        torch.cuda.synchronize()
    events = sorted((e for e in recorded.events()
                     if e.device_type == torch.autograd.DeviceType.CUDA),
                    key=lambda e: e.time_range.start)
    table = collections.OrderedDict()
    latest_end = None
    for event in events:
        name = event.name.replace("(anonymous namespace)::", "").replace("void ", "")
        name = name.split("(")[0][:56]
        row = table.setdefault(name, [0, 0.0, 0.0])
        begin, end = event.time_range.start, event.time_range.end
        row[0] += 1
        row[1] += end - begin
        row[2] += max(0.0, end - (begin if latest_end is None else max(begin, latest_end)))
        latest_end = end if latest_end is None else max(latest_end, end)
    span = events[-1].time_range.end - events[0].time_range.start
    print(f"{options.timeline}: {config.num_hidden_layers} layers, batch {batch}, "
          f"{length} tokens of context or prompt; {steps} step(s) span {span:.1f} us")
    print(f"{'launches':>8} {'mean us':>9} {'exclusive us':>12} {'sum excl us':>12}  kernel")
    for name, (count, total, exclusive) in table.items():
        print(f"{count:8d} {total / count:9.1f} {exclusive / count:12.1f} {exclusive:12.1f}  {name}")
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=192)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--layers", type=int, default=None,
                        help="run fewer layers of the same sizes (recorded in config)")
    parser.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    parser.add_argument("--profile", choices=("decode", "prefill"), default=None,
                        help="run one eager step of this kind between cudaProfilerStart/Stop "
                             "(for ncu --profile-from-start off) and print nothing else")
    parser.add_argument("--timeline", choices=("decode", "prefill", "mixed"), default=None,
                        help="print the kernels of the step with their times as they run in "
                             "place (CUPTI through torch.profiler) and nothing else")
    parser.add_argument("--prompt-len", type=int, default=PROMPT_LEN)
    parser.add_argument("--serving", type=int, default=0, metavar="REQUESTS",
                        help="run a continuous-batching workload of this many requests instead "
                             "and print its own JSON line")
    parser.add_argument("--shape", choices=tuple(SHAPES), default="llama-2-7b",
                        help="layer sizes for --serving, --profile and --timeline (the contract "
                             "line is always the Llama-2-7B shape)")
    parser.add_argument("--cache-fraction", type=float, default=0.5,
                        help="--serving: share of the memory left after the weights that the "
                             "cache pool takes")
    parser.add_argument("--log-dir", default=None,
                        help="where the clock samples of the timed region are kept "
                             "(default: a temporary folder)")
    options = parser.parse_args()
    if options.impl == "reference":
        return reference_arm()
    if options.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {options.gpus} is not supported")
        return 2
    if options.warmup < 3:
        options.warmup = 3
    special = bool(options.serving or options.profile or options.timeline)
    if options.shape != "llama-2-7b" and not special:
        print("bench.py: the contract line is measured at the Llama-2-7B shape; --shape goes with "
              "--serving, --profile or --timeline")
        return 2

    import numpy as np
    import torch

    from helix_runtime_b200 import Engine, EngineConfig, LlamaConfig, random_model
    from helix_runtime_b200.cache.manager import CacheManager
    from helix_runtime_b200.engine.step import StepEntry, StepFunction
    from helix_runtime_b200.ops import library as ops
    from helix_runtime_b200.sampling import Sampler

    peaks = load_peaks()
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    ops.lib()
    shape = dict(SHAPES[options.shape])
    if options.layers is None:
        options.layers = shape["num_hidden_layers"]
    shape["num_hidden_layers"] = options.layers
    config = LlamaConfig(**shape)
    model = random_model(config, seed=0, dtype="bfloat16", device=device)
    rng = np.random.default_rng(0)
    out_dir = options.log_dir or tempfile.mkdtemp(prefix="helix_bench_")
    os.makedirs(out_dir, exist_ok=True)
    steps, warmup = options.steps, options.warmup

    def fresh(batch: int, total_len: int, capacity: int):
        kv, state = model.cache_needs()
        pages = batch * -(-total_len // PAGE_SIZE) + 8
        cache = CacheManager(kv, state, PAGE_SIZE, pages, batch, config.max_position_embeddings,
                             model.dtype, device)
        step = StepFunction(model, cache, max_tokens=capacity, max_requests=batch)
        sampler = Sampler(device, max(batch, 1))
        return cache, step, sampler

    def timed(fn, count: int) -> float:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(count):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop)

    mean_context = PROMPT_LEN + GENERATED // 2

    def decode_through_engine(batch: int, n_steps: int, n_warmup: int, clock: str):
        """Decoding through the engine's own calls.  Each repeat: ``batch`` fresh requests whose
        prompts place the timed steps around the workload's mean context, their prompts and
        ``n_warmup`` decode steps untimed, then ``n_steps`` iterations timed with CUDA events
        (``clock="device"``) or with the host's clock between two synchronisations
        (``"host"``).  Repeats go on until a second has been timed.  Returns the per-step
        milliseconds of every repeat and what the engine says about its graphs."""
        # prompts are fed a few per iteration while the requests that came first already
        # decode: those are ahead by up to `feeding` tokens when the timed steps begin
        feeding = -(-batch * mean_context // PREFILL_TOKENS)
        prompt_len = max(16, mean_context - n_warmup - n_steps // 2 - feeding // 2)
        new_tokens = n_warmup + n_steps + feeding + 8
        rows = prompt_len + new_tokens
        engine = Engine(model, EngineConfig(
            page_size=PAGE_SIZE, max_running_requests=batch,
            max_tokens_per_iteration=PREFILL_TOKENS,
            num_pages=batch * -(-rows // PAGE_SIZE) + 8))
        per_step, contexts = [], []
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        while len(per_step) < 3 or sum(per_step) * n_steps < MIN_TIMED_SECONDS * 1e3:
            ids = [engine.submit([int(t) for t in rng.integers(0, config.vocab_size, prompt_len)],
                                 max_new_tokens=new_tokens) for _ in range(batch)]
            while any(engine.request(r).state.value != "decoding" for r in ids):
                engine.run_iteration()
            for _ in range(n_warmup):
                engine.run_iteration()
            torch.cuda.synchronize()
            sampled = 0
            contexts.append(sum(engine.cache.reserved(r) for r in ids) / batch + (n_steps + 1) / 2.0)
            if clock == "device":
                start.record()
                for _ in range(n_steps):
                    sampled += engine.run_iteration().sampled
                stop.record()
                torch.cuda.synchronize()
                elapsed_ms = start.elapsed_time(stop)
            else:
                begin = time.perf_counter()
                for _ in range(n_steps):
                    sampled += engine.run_iteration().sampled
                torch.cuda.synchronize()
                elapsed_ms = (time.perf_counter() - begin) * 1e3
            if sampled != batch * n_steps:
                raise RuntimeError(f"{sampled} tokens decoded in {n_steps} steps of batch {batch}")
            per_step.append(elapsed_ms / n_steps)
            for request_id in ids:
                engine.cancel(request_id)
            engine.run_until_done()              # the step that was queued ahead
            if len(per_step) >= 64:
                break
        kernels = max(engine.graphs.kernels_per_graph.values(), default=0)
        facts = {"prompt_len": prompt_len, "kernels_per_step": kernels,
                 "context_mean": sum(contexts) / len(contexts),
                 "graph_replays": engine.graphs.replays, "upload_bytes": engine.step_function.upload_bytes,
                 "steps_queued_ahead": engine.steps_queued_ahead}
        del engine
        torch.cuda.empty_cache()
        return per_step, facts

    weight_bytes = model.weight_bytes_per_step()
    kv_bytes_per_token = sum(2 * need.kv_heads * need.head_dim * 2
                             for need in model.cache_needs()[0].values())

    def hbm_fraction(batch: int, ms: float, context: float):
        """(bytes a decode step of this batch has to read, GB/s achieved, fraction of peak)"""
        step_bytes = weight_bytes + batch * context * kv_bytes_per_token
        achieved = step_bytes / (ms / 1e3) / 1e9
        return step_bytes, achieved, achieved / peaks["hbm_gbs"]

    def median(values):
        ordered = sorted(values)
        middle = len(ordered) // 2
        return ordered[middle] if len(ordered) % 2 else 0.5 * (ordered[middle - 1] + ordered[middle])

    if options.profile is not None:
        return profile_region(options, model, config, fresh, rng)
    if options.timeline is not None:
        return timeline_region(options, model, config, fresh, rng)
    if options.serving:
        return serving_workload(options, model, config, rng)

    # ------------------------------------------------------------------ prefill, 2,048 tokens
    # (first: a burst on a GPU that the decode loops have not yet driven into its power cap,
    # which is how the burst peak it is compared with was taken; the clock samples cover it
    # and the decode loop that follows)
    sampler_clock = ClockSampler(os.path.join(out_dir, "bench_clocks.csv"))
    sampler_clock.start()
    cache, step, sampler = fresh(1, PREFILL_TOKENS, PREFILL_TOKENS)
    prompt = [int(t) for t in rng.integers(0, config.vocab_size, PREFILL_TOKENS)]

    def prefill_once():
        cache.admit("p")
        step.run([StepEntry("p", prompt, [PREFILL_TOKENS - 1])], check_status=False)
        cache.release("p")

    for _ in range(3):
        prefill_once()
    reps = 5
    prefill_ms = timed(prefill_once, reps) / reps
    step.raise_on_status()
    h, i, layers, t = config.hidden_size, config.intermediate_size, options.layers, PREFILL_TOKENS
    prefill_flops = 2.0 * t * layers * (4 * h * h + 3 * h * i) + 2.0 * h * config.vocab_size \
        + 2.0 * layers * t * (t + 1) * h
    prefill_rate = prefill_flops / (prefill_ms / 1e3) / 1e12
    prefill = {"value": round(t / (prefill_ms / 1e3), 1), "tokens": t, "ms": round(prefill_ms, 3),
               "frac": round(prefill_rate / peaks["bf16_tflops"], 4),
               "frac_sustained": round(prefill_rate / peaks["bf16_tflops_sustained"], 4),
               "tflops": round(prefill_rate, 1)}
    del cache, step, sampler
    torch.cuda.empty_cache()

    # ------------------------------------------------------------------ decode, batch B
    repeats_ms, facts = decode_through_engine(options.batch, steps, warmup, "device")
    clocks = sampler_clock.stop()
    ms_per_step = median(repeats_ms)
    value = options.batch / (ms_per_step / 1e3)
    step_bytes, achieved_gbs, fraction = hbm_fraction(options.batch, ms_per_step, facts["context_mean"])
    roofline = {"bound": "hbm", "achieved": round(achieved_gbs, 1), "peak": peaks["hbm_gbs"],
                "unit": "GB/s", "frac": round(fraction, 4), "peak_source": peaks["source"]}

    # ------------------------------------------------------------------ end to end
    host_ms, host_facts = decode_through_engine(options.batch, steps, warmup, "host")
    e2e_ms = median(host_ms)
    e2e = {"value": round(options.batch / (e2e_ms / 1e3), 1), "unit": "tokens/s",
           "h2d_bytes_per_step": host_facts["upload_bytes"],
           "d2h_bytes_per_step": options.batch * 4 + 4,
           "ms_per_step": round(e2e_ms, 4), "repeats": len(host_ms),
           "graph_replays": host_facts["graph_replays"]}

    # ------------------------------------------------------------------ batch 1 and 64
    points = {}
    if not options.no_points:
        for batch in (1, 64):
            point_ms, point_facts = decode_through_engine(batch, steps, warmup, "device")
            point = median(point_ms)
            points[f"decode_b{batch}"] = round(batch / (point / 1e3), 1)
            points[f"decode_b{batch}_ms"] = round(point, 4)
            points[f"decode_b{batch}_frac"] = round(
                hbm_fraction(batch, point, point_facts["context_mean"])[2], 4)
            points[f"decode_b{batch}_context"] = round(point_facts["context_mean"], 1)

    kernels_per_step = facts["kernels_per_step"]
    line = {
        "metric": "decode tokens/s (Llama-2-7B shape, bf16, batch 8)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_per_step, 4), "ms_per_step_min": round(min(repeats_ms), 4),
        "ms_per_step_max": round(max(repeats_ms), 4), "repeats": len(repeats_ms),
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random N(0,0.02) weights from seed 0, uniform random token ids",
        "config": {"model": "llama-2-7b-shape", "layers": options.layers,
                   "layers_full": SHAPE["num_hidden_layers"], "hidden": h,
                   "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
                   "head_dim": config.head_dim, "intermediate": i, "vocab": config.vocab_size,
                   "global_batch": options.batch, "seq_len": PROMPT_LEN, "gen_len": GENERATED,
                   "timed_prompt_len": facts["prompt_len"], "timed_context_mean": round(facts["context_mean"], 1),
                   "context": config.max_position_embeddings, "page_size": PAGE_SIZE,
                   "parallelism": "single-gpu",
                   "l2": "each step streams >126MB of weights; no flush needed"},
        "e2e": e2e, "gpu_launches": int(kernels_per_step * steps * len(repeats_ms)),
        "kernels_per_step": int(kernels_per_step),
        "prefill": prefill, "roofline": roofline, "points": points, "clocks": clocks,
        "step_bytes": int(step_bytes), "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
