"""Generation through the Python entry point and the command line, against the plain
implementation: greedy and temperature sampling, many requests with chunked prompts mixed
with decoding, stop reasons and the count of cached tokens."""
from __future__ import annotations

import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, random_tokens
from helix_runtime_b200 import Engine
from helix_runtime_b200.sampling import uniform_for
from tiny_configs import PAGE_SIZE, tiny_config

pytestmark = pytest.mark.gpu

SLACK = {"float32": 1e-4, "bfloat16": 6e-3}


def check_greedy(plain, prompt, generated, dtype):
    """Teacher-forced: every generated token is a maximum of the plain logits for the prefix
    the engine itself produced, up to the precision of the dtype."""
    tokens = list(prompt)
    for index, token in enumerate(generated):
        row = plain.logits(tokens)[-1]
        assert row[token] >= row.max() - SLACK[dtype], \
            f"token {index}: engine chose {token}, plain prefers {int(np.argmax(row))}"
        tokens.append(token)


def check_sampled(plain, prompt, generated, temperature, seed, dtype):
    tokens = list(prompt)
    for index, token in enumerate(generated):
        row = plain.logits(tokens)[-1].astype(np.float64)
        weights = np.exp((row - row.max()) / temperature)
        cumulative = np.cumsum(weights) / weights.sum()
        u = uniform_for(seed, index)
        want = min(int(np.searchsorted(cumulative, u, side="right")), len(row) - 1)
        if token != want:
            # the engine's logits differ from the plain ones by rounding: the draw may fall on
            # the other side of a boundary that lies that close to u
            low, high = sorted((token, want))
            margin = 20 * SLACK[dtype] / temperature
            assert high - low <= 2 and abs(cumulative[low] - u) < margin, \
                f"token {index}: engine drew {token}, plain draws {want} (u={u})"
        tokens.append(token)


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"),
                                        ("A", "bfloat16"), ("B", "bfloat16"),
                                        ("C", "bfloat16")])
def test_greedy_generation(name, dtype, folders, plain_models):
    plain = plain_models(name, dtype)
    vocab = tiny_config(name).vocab_size
    engine = Engine.from_pretrained(folders(name, dtype), dtype=dtype, page_size=PAGE_SIZE[name],
                                    max_running_requests=4, max_tokens_per_iteration=64)
    prompts = [random_tokens(vocab, length, seed=length) for length in (5, 17, 31)]
    results = engine.generate(prompts, max_new_tokens=12)
    for prompt, result in zip(prompts, results):
        assert len(result.generated_tokens) == 12 and result.stop_reason == "max_new_tokens"
        assert result.cached_token_count == len(prompt) + 12 - 1
        check_greedy(plain, prompt, result.generated_tokens, dtype)
    if dtype == "float32":
        assert results[1].generated_tokens == plain.greedy(prompts[1], 12)
    engine.cache.check()
    assert not engine.cache.live_requests()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_requests_chunked_prompts_mixed_with_decoding(dtype, folders, plain_models):
    """Tiny B's workload: prompts of 1/9/40/64/100 tokens, 20 new tokens, temperature 0.8 at a
    fixed seed plus a greedy run, prompts cut at 32 tokens and mixed with decode tokens."""
    plain = plain_models("B", dtype)
    prompts = [random_tokens(384, length, seed=200 + length) for length in (1, 9, 40, 64, 100)]
    engine = Engine.from_pretrained(folders("B", dtype), dtype=dtype, page_size=16,
                                    max_running_requests=4, max_tokens_per_iteration=48,
                                    max_prefill_chunk=32, num_pages=24, poison_free_pages=True)
    greedy = engine.generate(prompts, max_new_tokens=20)
    for prompt, result in zip(prompts, greedy):
        check_greedy(plain, prompt, result.generated_tokens, dtype)
    sampled = engine.generate(prompts, max_new_tokens=20, temperature=0.8, seed=11)
    for index, (prompt, result) in enumerate(zip(prompts, sampled)):
        assert len(result.generated_tokens) == 20
        check_sampled(plain, prompt, result.generated_tokens, 0.8, 11 + index, dtype)
    assert any(a.generated_tokens != b.generated_tokens for a, b in zip(greedy, sampled))
    again = engine.generate(prompts, max_new_tokens=20, temperature=0.8, seed=11)
    assert [r.generated_tokens for r in again] == [r.generated_tokens for r in sampled]
    stats = engine.stats()
    assert stats["scheduler"]["prefill_tokens"] > 0 and stats["scheduler"]["decode_tokens"] > 0
    assert stats["cache"]["groups"][0]["reuses"] > 0
    engine.cache.check()


@pytest.mark.parametrize("name,dtype", [("C", "bfloat16"), ("B", "float32")])
@pytest.mark.parametrize("live", [24, 64, 100])
def test_decode_steps_with_dozens_of_live_requests(name, dtype, live, folders, plain_models):
    """24, 64 and 100 requests decode together (64 is the benchmark's largest batch): above 16
    tokens a step the streaming attention is launched by another protocol and the
    weight-streaming products take wider token tiles, up to 128 tokens, the widest, with 100.
    Half as many requests again wait for a slot, so pages
    and slots are used again; every token of every request is checked."""
    plain = plain_models(name, dtype)
    config = tiny_config(name)
    page = PAGE_SIZE[name]
    total = live + live // 2
    rng = np.random.default_rng(live)
    lengths = [int(n) for n in rng.integers(1, 40, size=total)]
    lengths[0], lengths[1], lengths[2] = 1, page, page + 1
    prompts = [random_tokens(config.vocab_size, n, seed=1000 + i) for i, n in enumerate(lengths)]
    new_tokens = 6
    pages_each = -(-(max(lengths) + new_tokens) // page)
    engine = Engine.from_pretrained(folders(name, dtype), dtype=dtype, page_size=page,
                                    max_running_requests=live, max_tokens_per_iteration=256,
                                    num_pages=live * pages_each, poison_free_pages=True)
    results = engine.generate(prompts, max_new_tokens=new_tokens)
    for prompt, result in zip(prompts, results):
        assert len(result.generated_tokens) == new_tokens
        check_greedy(plain, prompt, result.generated_tokens, dtype)
    stats = engine.stats()
    assert stats["cache"]["groups"][0]["reuses"] > 0
    assert stats["scheduler"]["decode_tokens"] >= total * (new_tokens - 1)
    # steps with more than 16 single-token requests did run
    assert engine.step_function.tokens_run / max(engine.step_function.steps_run, 1) > 16
    engine.cache.check()
    assert not engine.cache.live_requests()


def test_a_context_that_crosses_two_graph_buckets(folders, plain_models):
    """Decode graphs are recorded for contexts rounded up to 256, 512, ...: a request that
    decodes from position 240 to the model's last position, 511, leaves the first bucket for
    the second while two shorter requests decode beside it, so two graphs are recorded and
    replayed; tokens around the border and every seventh token elsewhere are checked."""
    plain = plain_models("C", "bfloat16")
    prompts = [random_tokens(512, n, seed=50 + n) for n in (240, 9, 130)]
    engine = Engine.from_pretrained(folders("C", "bfloat16"), dtype="bfloat16", page_size=16,
                                    max_running_requests=3, max_tokens_per_iteration=256)
    ids = [engine.submit(prompts[0], 272), engine.submit(prompts[1], 272),
           engine.submit(prompts[2], 272)]
    engine.run_until_done()
    assert engine.graphs.captures >= 2 and engine.graphs.replays > 200
    for request_id, prompt in zip(ids, prompts):
        generated = engine.request(request_id).generated
        assert len(generated) == 272
        # teacher-forced check of every 7th token and of the tokens around the bucket borders
        full = prompt + generated
        logits = plain.logits(full[:-1])
        for index in range(len(generated)):
            position = len(prompt) + index - 1
            near_border = abs(position + 1 - 256) <= 3 or position >= 508
            if index % 7 and not near_border:
                continue
            row = logits[position]
            assert row[generated[index]] >= row.max() - SLACK["bfloat16"], (request_id, index)


def test_stop_reasons_and_cached_token_count(folders, plain_models):
    plain = plain_models("A", "float32")
    engine = Engine.from_pretrained(folders("A", "float32"), dtype="float32", page_size=8,
                                    max_running_requests=2, max_tokens_per_iteration=64)
    prompt = random_tokens(256, 6, seed=1)
    free_run = engine.generate([prompt], max_new_tokens=8)[0].generated_tokens
    eos = free_run[3]
    first = free_run.index(eos)
    result = engine.generate([prompt], max_new_tokens=8, eos_token=eos)[0]
    assert result.stop_reason == "eos_token" and result.generated_tokens == free_run[:first + 1]
    assert result.cached_token_count == len(prompt) + first      # the eos token is not fed back
    long_prompt = random_tokens(256, 126, seed=2)
    result = engine.generate([long_prompt], max_new_tokens=10)[0]
    assert result.stop_reason == "context_limit" and len(result.generated_tokens) == 3
    assert result.cached_token_count == 128
    check_greedy(plain, long_prompt, result.generated_tokens, "float32")
    result = engine.generate([prompt], max_new_tokens=0)[0]
    assert result.generated_tokens == [] and result.cached_token_count == len(prompt)


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16")])
def test_prompts_that_begin_alike_share_pages_and_generate_the_same(name, dtype, folders,
                                                                    plain_models):
    """With the prefix index on, later requests adopt the pages of a common beginning and run
    only the rest of their prompt; what they generate is checked against the plain
    implementation exactly as without sharing.  The pool is small, so kept prefixes are also
    dropped under pressure while others are still being shared."""
    plain = plain_models(name, dtype)
    vocab = tiny_config(name).vocab_size
    page = PAGE_SIZE[name]
    stem = random_tokens(vocab, 3 * page + 3, seed=77)
    prompts = [stem + random_tokens(vocab, extra, seed=100 + extra) for extra in (2, 9, 1, 20)]
    prompts.insert(2, stem[:2 * page + 1] + random_tokens(vocab, 4, seed=6))  # shares two pages
    prompts.append(random_tokens(vocab, 4 * page, seed=5))                    # shares nothing
    engine = Engine.from_pretrained(folders(name, dtype), dtype=dtype, page_size=page,
                                    max_running_requests=2, max_tokens_per_iteration=48,
                                    num_pages=14, poison_free_pages=True,
                                    prefix_cache_entries=3)
    results = []
    for prompt in prompts:        # one after the other, so that each finds what the last left
        results += engine.generate([prompt], max_new_tokens=6)
    for prompt, result in zip(prompts, results):
        check_greedy(plain, prompt, result.generated_tokens, dtype)
    stats = engine.stats()
    assert stats["prefix"]["hits"] >= 4
    assert stats["prefix"]["reused_tokens"] >= 3 * (3 * page) + 2 * page
    assert [engine.request(i).reused_tokens for i in range(6)] == \
        [0, 3 * page, 2 * page, 3 * page, 3 * page, 0]
    # requests that ran together while sharing: same answers
    together = engine.generate(prompts[:4], max_new_tokens=6)
    for prompt, result in zip(prompts, together):
        check_greedy(plain, prompt, result.generated_tokens, dtype)
    engine.cache.check()
    # a request may keep out of the index
    before = engine.stats()["prefix"]["lookups"]
    engine.generate([prompts[0]], max_new_tokens=2, cache_namespace=None)
    assert engine.stats()["prefix"]["lookups"] == before
    engine.prefix.clear()
    engine.cache.check()
    assert all(group.pool.pages_in_use == 0 for group in engine.cache.groups)


def run_requests(engine, prompts, budgets, eos, temperatures, cancel_after=None):
    ids = [engine.submit(prompt, max_new_tokens=budget, eos_token=eos, temperature=temperature,
                         seed=40 + index)
           for index, (prompt, budget, temperature) in enumerate(zip(prompts, budgets, temperatures))]
    iterations = 0
    while engine.scheduler.has_unfinished() or engine._flight is not None:
        engine.run_iteration()
        iterations += 1
        if cancel_after is not None and iterations == cancel_after[0]:
            assert engine.cancel(ids[cancel_after[1]])
            engine.cache.check()
    engine.cache.check()
    assert not engine.cache.live_requests()
    return [(list(engine.request(i).generated), engine.request(i).stop_reason.value,
             engine._cached_at_finish.get(i)) for i in ids]


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("C", "bfloat16")])
def test_steps_queued_ahead_change_nothing(name, dtype, folders, plain_models):
    """The engine queues the next decode step before it has read the tokens of the one in
    flight.  Requests that end at different times (an end-of-sequence token nobody could
    foresee, their count of new tokens, the context limit), greedy and sampled, more requests
    than run at once and a pool that makes them wait: token for token, stop reason and cached
    count as without looking ahead, and as the plain implementation says."""
    plain = plain_models(name, dtype)
    config = tiny_config(name)
    page = PAGE_SIZE[name]
    limit = config.max_position_embeddings
    prompts = [random_tokens(config.vocab_size, length, seed=300 + length)
               for length in (5, 33, 12, limit - 6, 20, 3)]
    budgets = [24, 40, 7, 30, 18, 33]
    temperatures = [0.0, 0.7, 0.0, 0.0, 0.9, 0.0]
    # token for token between two runs: the bfloat16 engine is asked for sums in a fixed order
    # (split-K atomics would leave a greedy pick between near-equal logits to chance)
    options = dict(dtype=dtype, page_size=page, max_running_requests=3,
                   max_tokens_per_iteration=64, num_pages=-(-limit // page) + 8,
                   poison_free_pages=True, ordered_sums=dtype == "bfloat16")
    free = Engine.from_pretrained(folders(name, dtype), lookahead=False, **options)
    free_run = run_requests(free, prompts, budgets, None, temperatures)
    eos = free_run[0][0][9]                     # the first request meets it at its tenth token
    outcomes = {}
    for lookahead in (False, True):
        engine = Engine.from_pretrained(folders(name, dtype), lookahead=lookahead, **options)
        outcomes[lookahead] = run_requests(engine, prompts, budgets, eos, temperatures)
        ahead = engine.stats()["steps_queued_ahead"]
        assert (ahead > 20) if lookahead else (ahead == 0)
    assert outcomes[True] == outcomes[False]
    reasons = [reason for _, reason, _ in outcomes[True]]
    assert reasons[0] == "eos_token" and "max_new_tokens" in reasons and reasons[3] == "context_limit"
    for prompt, temperature, (generated, _, _) in zip(prompts, temperatures, outcomes[True]):
        if temperature == 0.0:
            check_greedy(plain, prompt, generated, dtype)
    # a request cancelled while its row of the step queued ahead is in flight
    engine = Engine.from_pretrained(folders(name, dtype), lookahead=True, **options)
    cancelled = run_requests(engine, prompts, budgets, eos, temperatures, cancel_after=(6, 1))
    assert cancelled[1][1] == "cancelled"
    for index in (0, 2):                         # those that ran beside it are untouched
        assert cancelled[index] == outcomes[True][index]


def test_ordered_sums_repeat_bit_for_bit(folders, plain_models):
    """With ``ordered_sums`` the decode products are not cut along the reduction, so nothing is
    summed by atomic adds: the same steps give the same logits to the last bit on a second
    run, and they are the plain implementation's within the usual tolerance."""
    from engine_harness import assert_close, tolerance
    from helix_runtime_b200 import StepEntry, StepFunction, load_model
    from helix_runtime_b200.cache.manager import CacheManager
    plain = plain_models("C", "bfloat16")
    a = random_tokens(512, 90, seed=1)
    b = random_tokens(512, 37, seed=2)
    runs = []
    for _ in range(2):
        model = load_model(folders("C", "bfloat16"), "bfloat16", "cuda:0")
        kv, state = model.cache_needs()
        cache = CacheManager(kv, state, 16, 16, 2, model.max_positions, model.dtype, model.device)
        step = StepFunction(model, cache, max_tokens=128, max_requests=2, ordered_sums=True)
        cache.admit("a")
        cache.admit("b")
        rows = [step.run([StepEntry("a", a[:70], [69]), StepEntry("b", b[:20], [19])])
                .cpu().numpy().copy()]
        for index in range(17):
            rows.append(step.run([StepEntry("a", [a[70 + index]], [0]),
                                  StepEntry("b", [b[20 + index]], [0])]).cpu().numpy().copy())
        runs.append(np.concatenate(rows))
    assert np.array_equal(runs[0], runs[1])
    expected_a, expected_b = plain.logits(a[:87]), plain.logits(b[:37])
    want = [expected_a[69], expected_b[19]]
    for index in range(17):
        want += [expected_a[70 + index], expected_b[20 + index]]
    assert_close(runs[0], np.stack(want), "ordered sums", **tolerance("bfloat16", "C"))


def test_graphs_recorded_before_the_scratch_grew_stay_valid(folders, plain_models):
    """A decode graph is recorded while the attention scratch is small; a large mixed step then
    makes the scratch grow (the float32 kernel keeps a part per key split of every row),
    further graphs are recorded, the allocator is told to hand unused memory back to the
    driver, and the first graph is replayed again.  The buffer it points at must still be
    there."""
    plain = plain_models("B", "float32")
    vocab = tiny_config("B").vocab_size
    engine = Engine.from_pretrained(folders("B", "float32"), dtype="float32", page_size=16,
                                    max_running_requests=6, max_tokens_per_iteration=2048,
                                    attention_split_keys=32, lookahead=False)
    first_prompt = random_tokens(vocab, 40, seed=1)
    first = engine.submit(first_prompt, max_new_tokens=40)
    for _ in range(6):
        engine.run_iteration()                       # alone: the one-token graph is recorded
    workspace = engine.step_function.workspace
    before = workspace.bytes()
    others = [engine.submit(random_tokens(vocab, 200, seed=10 + index), max_new_tokens=4)
              for index in range(4)]
    while any(not engine.request(other).is_terminal for other in others):
        engine.run_iteration()                       # mixed step, five-token graphs
    torch.cuda.empty_cache()
    engine.run_until_done()                          # alone again: the first graph
    assert workspace._retired, "the scratch did not grow: the test no longer tests anything"
    assert workspace.bytes() > before
    assert engine.graphs.captures >= 2 and engine.graphs.replays > 20
    check_greedy(plain, first_prompt, engine.request(first).generated, "float32")
    for index, request in enumerate(others):
        check_greedy(plain, random_tokens(vocab, 200, seed=10 + index),
                     engine.request(request).generated, "float32")
    engine.cache.check()


def test_everything_at_once_under_page_pressure(folders, plain_models):
    """Twenty requests with prompts of 20 to 300 tokens, half of them with a common beginning,
    over a pool that holds three of them: requests wait, are preempted and recomputed, kept
    prefixes are dropped under pressure, decode steps are replayed as graphs for ever new
    subsets of requests and queued ahead where that is possible.  Every greedy token must be
    the plain implementation's."""
    plain = plain_models("C", "bfloat16")
    vocab = tiny_config("C").vocab_size
    rng = np.random.default_rng(5)
    stem = random_tokens(vocab, 64, seed=99)
    prompts = []
    for index in range(20):
        body = random_tokens(vocab, int(rng.integers(20, 301)), seed=400 + index)
        prompts.append(stem + body if index % 2 == 0 else body)
    engine = Engine.from_pretrained(folders("C", "bfloat16"), dtype="bfloat16", page_size=16,
                                    max_running_requests=8, max_tokens_per_iteration=512,
                                    max_prefill_chunk=128, num_pages=64, poison_free_pages=True,
                                    prefix_cache_entries=4)
    ids = [engine.submit(prompt, max_new_tokens=24, cache_namespace="x") for prompt in prompts]
    engine.run_until_done()
    engine.cache.check()
    stats = engine.stats()
    assert stats["scheduler"]["finished"] == 20 and stats["scheduler"]["failed"] == 0
    assert stats["scheduler"]["preemptions"] > 0 and stats["scheduler"]["kv_limited_iterations"] > 0
    assert stats["prefix"]["hits"] > 0 and stats["steps_queued_ahead"] > 0
    assert engine.graphs.captures > 3
    for prompt, request in zip(prompts, ids):
        generated = engine.request(request).generated
        assert len(generated) == 24
        check_greedy(plain, prompt, generated, "bfloat16")
    metrics = engine.metrics()
    assert metrics.finished_count == 20 and metrics.generated_tokens == 20 * 24
    assert metrics.time_to_first_token.sample_count == 20
    assert metrics.inter_token_latency.sample_count == 20 * 23
    assert metrics.throughput_defined and metrics.generated_tokens_per_second > 0.0
    assert metrics.waiting_time.maximum_seconds <= metrics.request_latency.maximum_seconds
    engine.prefix.clear()
    assert all(group.pool.pages_in_use == 0 for group in engine.cache.groups)


def test_the_pool_can_be_sized_from_free_memory(folders, plain_models):
    import torch
    free_bytes, _ = torch.cuda.mem_get_info()
    engine = Engine.from_pretrained(folders("A", "float32"), dtype="float32", page_size=8,
                                    max_running_requests=2, cache_memory_fraction=0.001)
    group = engine.cache.groups[0]
    page_bytes = 2 * 2 * 4 * 16 * 4 * 8      # layers, keys and values, heads, head size, float32, page
    assert abs(group.pool.num_pages * page_bytes - 0.001 * free_bytes) < 0.1 * 0.001 * free_bytes
    prompt = [1, 42, 17, 5, 9]
    assert engine.generate([prompt], max_new_tokens=6)[0].generated_tokens == \
        plain_models("A", "float32").greedy(prompt, 6)
    with pytest.raises(ValueError, match="cache_memory_fraction"):
        Engine.from_pretrained(folders("A", "float32"), dtype="float32", cache_memory_fraction=1.5)


def test_bad_submissions_are_refused(folders):
    engine = Engine.from_pretrained(folders("A", "float32"), dtype="float32", page_size=8,
                                    max_running_requests=2, num_pages=4)
    with pytest.raises(ValueError, match="vocabulary"):
        engine.submit([1, 256])
    with pytest.raises(ValueError, match="eos token"):
        engine.submit([1], eos_token=999)
    with pytest.raises(ValueError, match="positions"):
        engine.submit([1] * 129)
    with pytest.raises(ValueError, match="never run"):
        engine.submit([1] * 30, max_new_tokens=10)       # 39 rows > 4 pages of 8
    with pytest.raises(ValueError, match="at least one"):
        engine.submit([])


def test_no_cpu_path():
    with pytest.raises(RuntimeError, match="no CPU path"):
        Engine.from_pretrained("/nonexistent", device="cpu")


def test_command_line(folders, plain_models):
    folder = folders("A", "float32")
    plain = plain_models("A", "float32")
    prompt = [1, 42, 17, 5, 9]
    completed = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "helix_generate"), "--model", folder,
         "--dtype", "float32", "--max-new-tokens", "6", "--page-size", "8", *map(str, prompt)],
        capture_output=True, text=True, cwd=ROOT)
    assert completed.returncode == 0, completed.stderr
    lines = completed.stdout.strip().splitlines()
    assert lines[0].startswith("generated_token_ids:")
    generated = [int(t) for t in lines[0].split(":", 1)[1].split()]
    assert generated == plain.greedy(prompt, 6)
    assert lines[1] == "stop_reason: max_new_tokens"
    assert lines[2] == "cached_token_count: 10"        # 5 + 6 - 1, as the reference counts
    failed = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "helix_generate"), "--model", folder,
         "--dtype", "float32", "999999"], capture_output=True, text=True, cwd=ROOT)
    assert failed.returncode == 1 and "helix_generate:" in failed.stderr


# -------------------------------------------------------------- Helix's native model file

GOLDEN = os.path.join(ROOT, "tests", "golden")


def test_reference_made_model_file_generates_the_references_tokens():
    """``tests/golden/tiny_A.helix`` was packed by the reference's own tools, and
    ``tiny_A.json`` holds what the reference's CPU model made of it: its greedy tokens and its
    last-position logits.  The float32 engine must give the same from the same file."""
    import json
    from helix_runtime_b200 import StepEntry, StepFunction, load_model
    from helix_runtime_b200.cache.manager import CacheManager
    with open(os.path.join(GOLDEN, "tiny_A.json"), "r", encoding="utf-8") as source:
        golden = json.load(source)
    path = os.path.join(GOLDEN, "tiny_A.helix")
    engine = Engine.from_pretrained(path, dtype="float32", page_size=8, max_running_requests=2)
    greedy = golden["greedy"]
    prompt = golden["tokens"][:greedy["prompt_length"]]
    result = engine.generate([prompt], max_new_tokens=len(greedy["tokens"]))[0]
    assert result.generated_tokens == greedy["tokens"]
    assert result.cached_token_count == len(prompt) + len(greedy["tokens"]) - 1
    # logits, in both precisions (bfloat16 at the tolerance of the other bfloat16 tests)
    for dtype, atol in (("float32", 2e-5), ("bfloat16", 5e-3)):
        model = load_model(path, dtype, "cuda:0")
        kv, state = model.cache_needs()
        cache = CacheManager(kv, state, 8, 16, 1, model.max_positions, model.dtype, model.device)
        step = StepFunction(model, cache, max_tokens=64, max_requests=1)
        for length, values in golden["last_logits_hex"].items():
            reference = np.asarray([float.fromhex(v) for v in values], dtype=np.float32)
            cache.admit("r")
            tokens = golden["tokens"][:int(length)]
            logits = step.run([StepEntry("r", tokens, [len(tokens) - 1])])
            np.testing.assert_allclose(logits.cpu().numpy()[0], reference, rtol=1e-4, atol=atol,
                                       err_msg=f"{dtype}, prefix of {length}")
            cache.release("r")


def test_command_line_and_replay_take_a_model_file(tmp_path):
    import json
    with open(os.path.join(GOLDEN, "tiny_A.json"), "r", encoding="utf-8") as source:
        golden = json.load(source)
    path = os.path.join(GOLDEN, "tiny_A.helix")
    greedy = golden["greedy"]
    prompt = golden["tokens"][:greedy["prompt_length"]]
    completed = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "helix_generate"), "--model", path,
         "--dtype", "float32", "--max-new-tokens", str(len(greedy["tokens"])), "--page-size", "8",
         *map(str, prompt)], capture_output=True, text=True, cwd=ROOT)
    assert completed.returncode == 0, completed.stderr
    generated = [int(t) for t in completed.stdout.splitlines()[0].split(":", 1)[1].split()]
    assert generated == greedy["tokens"]
    # replay: the last position of the longest golden prefix, fed in two portions
    length = max(int(key) for key in golden["last_logits_hex"])
    tokens = golden["tokens"][:length]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:11], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[11:],
                                      "want": [length - 12]}], "end": ["a"]}]
    out_dir = tmp_path / "replay"
    replay = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", path, "--dtype",
         "float32", "--out", str(out_dir), "--max-tokens", "64", "--page-size", "8"],
        input="".join(json.dumps(step) + "\n" for step in steps), capture_output=True, text=True,
        cwd=ROOT)
    assert replay.returncode == 0, replay.stderr
    got = np.fromfile(out_dir / "1.f32", dtype="<f4")
    reference = np.asarray([float.fromhex(v) for v in golden["last_logits_hex"][str(length)]],
                           dtype=np.float32)
    np.testing.assert_allclose(got, reference, rtol=1e-4, atol=2e-5)
    # a damaged file is refused with the reader's message, exit code 1
    damaged = tmp_path / "damaged.helix"
    data = bytearray(open(path, "rb").read())
    data[4000] ^= 0x01
    damaged.write_bytes(bytes(data))
    failed = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "helix_generate"), "--model", str(damaged),
         "--dtype", "float32", "1", "2"], capture_output=True, text=True, cwd=ROOT)
    assert failed.returncode == 1 and "checksum mismatch" in failed.stderr
