"""Failure paths through the engine, every failure made on the host.

Nothing here faults, traps or hangs the GPU: a NaN is written into a weight, the status word
is set with an ordinary fill, and the one wait that runs out is a wait of a few thousand polls
on a barrier nobody arrives at, after which its kernel returns (the reference injects its
failure the same way, a NaN in the output head, tests/cpu_runtime_engine_test.cpp:498-520).
"""
from __future__ import annotations

import pytest
import torch

from conftest import random_tokens
from helix_runtime_b200 import Engine
from helix_runtime_b200.engine import RequestState
from helix_runtime_b200.ops import library as ops
from tiny_configs import PAGE_SIZE, tiny_config

pytestmark = pytest.mark.gpu


def all_pages_free(engine) -> bool:
    engine.cache.check()
    return engine.cache.free_pages() == [group.pool.num_pages for group in engine.cache.groups] \
        and engine.cache.free_slots == engine.cache.max_requests


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_requests_nan_fails_that_request_only(dtype, folders, plain_models):
    """A NaN in the embedding row of a token that one request alone feeds: that request fails
    with a non-finite message at its first sampling, the others in the same batch generate
    what the plain implementation generates, every page comes back."""
    plain = plain_models("A", dtype)
    engine = Engine.from_pretrained(folders("A", dtype), dtype=dtype, page_size=PAGE_SIZE["A"],
                                    max_running_requests=4, max_tokens_per_iteration=64)
    poisoned_token = 255
    prompts = [[t for t in random_tokens(255, length, seed=10 + length)]     # ids below 255
               for length in (9, 14, 5)]
    bad_prompt = prompts[1][:6] + [poisoned_token] + prompts[1][6:]
    table = engine.model.embedding.table
    saved = table[poisoned_token].clone()
    table[poisoned_token, 3] = float("nan")
    ids = [engine.submit(prompts[0], 5), engine.submit(bad_prompt, 5), engine.submit(prompts[2], 5)]
    engine.run_until_done()
    states = [engine.request(i).state for i in ids]
    assert states == [RequestState.FINISHED, RequestState.FAILED, RequestState.FINISHED]
    assert "non-finite" in engine.request(ids[1]).error
    assert engine.request(ids[1]).generated == []
    for request_id, prompt in ((ids[0], prompts[0]), (ids[2], prompts[2])):
        generated = engine.request(request_id).generated
        tokens = list(prompt)
        for token in generated:
            row = plain.logits(tokens)[-1]
            assert row[token] >= row.max() - (1e-4 if dtype == "float32" else 6e-3)
            tokens.append(token)
        assert len(generated) == 5
    assert all_pages_free(engine)
    assert engine.stats()["scheduler"]["failed"] == 1
    # repaired: the same prompt runs
    table[poisoned_token] = saved
    again = engine.generate([bad_prompt], max_new_tokens=3)[0]
    assert len(again.generated_tokens) == 3 and all_pages_free(engine)


def test_nan_in_the_output_head_fails_every_request_and_the_engine_goes_on(folders):
    engine = Engine.from_pretrained(folders("B", "float32"), dtype="float32",
                                    page_size=PAGE_SIZE["B"], max_running_requests=3)
    head = engine.model.lm_head.weight.matrix
    saved = head[7].clone()
    head[7, 11] = float("nan")              # logit 7 of every row becomes NaN
    ids = [engine.submit(random_tokens(384, n, seed=n), 4) for n in (3, 20)]
    engine.run_until_done()
    for request_id in ids:
        request = engine.request(request_id)
        assert request.state is RequestState.FAILED and "non-finite" in request.error
    with pytest.raises(RuntimeError, match="failed: logits contain a non-finite value"):
        engine.generate([[1, 2, 3]], max_new_tokens=2)
    assert all_pages_free(engine)
    head[7] = saved
    assert len(engine.generate([[1, 2, 3]], max_new_tokens=2)[0].generated_tokens) == 2
    assert all_pages_free(engine)


def test_a_flagged_step_fails_the_step_queued_behind_it(folders):
    """The status word is raised from the host while decode steps are queued ahead of their
    predecessors' completion: the step that reports it fails, the step queued behind it fails
    with it, what both had reserved goes back, and the engine serves the next submission."""
    engine = Engine.from_pretrained(folders("C", "bfloat16"), dtype="bfloat16",
                                    page_size=PAGE_SIZE["C"], max_running_requests=2)
    assert engine.config.lookahead and engine.graphs is not None
    ids = [engine.submit(random_tokens(512, n, seed=n), 40) for n in (30, 12)]
    while engine._flight is None:                       # until a step is queued ahead
        assert not engine.run_iteration().idle
    generated_before = [len(engine.request(i).generated) for i in ids]
    engine.step_function.status.fill_(ops.FLAG_WAIT_TIMEOUT)
    iterations = engine.run_until_done()
    assert iterations <= 3                              # no further steps were started
    for request_id, before in zip(ids, generated_before):
        request = engine.request(request_id)
        assert request.state is RequestState.FAILED
        assert "a bounded kernel wait ran out" in request.error
        assert len(request.generated) <= before + 1     # at most the step already in flight
    assert engine._flight is None and all_pages_free(engine)
    assert int(engine.step_function.status.item()) == 0
    result = engine.generate([random_tokens(512, 9, seed=3)], max_new_tokens=6)[0]
    assert len(result.generated_tokens) == 6 and all_pages_free(engine)


def test_a_page_flag_fails_the_step_and_rolls_its_reservation_back(folders):
    engine = Engine.from_pretrained(folders("A", "float32"), dtype="float32",
                                    page_size=PAGE_SIZE["A"], max_running_requests=2,
                                    cuda_graphs=False)
    request_id = engine.submit(random_tokens(256, 20, seed=1), 8)
    engine.run_iteration()                               # the prompt
    assert engine.request(request_id).state is RequestState.DECODING
    engine.step_function.status.fill_(ops.FLAG_BAD_PAGE)
    engine.run_iteration()
    request = engine.request(request_id)
    assert request.state is RequestState.FAILED and "block table entry" in request.error
    assert all_pages_free(engine)


def test_scheduler_and_cache_must_agree_on_where_a_request_stands(folders):
    """The step takes token values from the scheduler's count and positions from the cache's;
    if the two ever disagree the step is refused instead of run at shifted positions."""
    engine = Engine.from_pretrained(folders("A", "float32"), dtype="float32",
                                    page_size=PAGE_SIZE["A"], max_running_requests=2,
                                    cuda_graphs=False)
    request_id = engine.submit(random_tokens(256, 11, seed=2), 8)
    engine.run_iteration()
    engine.scheduler.request(request_id).processed -= 1          # a fault made by hand
    engine.run_iteration()
    request = engine.request(request_id)
    assert request.state is RequestState.FAILED
    assert "the scheduler feeds tokens from 10, the cache stands at 11" in request.error
    assert all_pages_free(engine)


def test_a_bounded_wait_that_runs_out_sets_the_flag_and_the_kernel_returns():
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    # somebody arrives: the wait succeeds, no flag
    assert ops.bounded_wait_check(2000, True, status) is True
    assert int(status.item()) == 0
    # nobody arrives: the wait gives up after its limit, flags it, and the kernel exits
    assert ops.bounded_wait_check(2000, False, status) is False
    assert int(status.item()) == ops.FLAG_WAIT_TIMEOUT
    # the device is as usable as before
    status.zero_()
    assert ops.bounded_wait_check(5, True, status) is True and int(status.item()) == 0
    with pytest.raises(ops.KernelError, match="polls"):
        ops.bounded_wait_check(10 ** 9, False, status)


def test_pages_of_a_request_cancelled_in_flight_wait_for_the_step_that_uses_them(folders,
                                                                                  plain_models):
    """A request cancelled while a decode step with its row is queued on the device: its pages
    and slot are parked, reach nobody until that step has completed, and the request beside
    it generates what the plain implementation generates."""
    plain = plain_models("C", "bfloat16")
    engine = Engine.from_pretrained(folders("C", "bfloat16"), dtype="bfloat16",
                                    page_size=PAGE_SIZE["C"], max_running_requests=2,
                                    num_pages=12)
    prompts = [random_tokens(512, n, seed=70 + n) for n in (33, 21)]
    ids = [engine.submit(prompt, 24) for prompt in prompts]
    while engine._flight is None:
        engine.run_iteration()
    free_before = engine.cache.free_pages()
    assert engine.cancel(ids[0])
    cache = engine.stats()["cache"]
    assert cache["parked_pages"] >= 3 and engine.cache.free_pages() == free_before
    assert not engine.cache.has(ids[0]) and engine.cache.free_slots == 0
    engine.cache.check()
    engine.run_iteration()                        # completes the step that was queued
    assert engine.stats()["cache"]["parked_pages"] == 0
    assert engine.cache.free_pages()[0] >= free_before[0] + 3
    late = engine.submit(random_tokens(512, 40, seed=5), 6)     # takes the parked slot and pages
    engine.run_until_done()
    assert engine.request(ids[0]).state is RequestState.CANCELLED
    for request_id, prompt in ((ids[1], prompts[1]), (late, random_tokens(512, 40, seed=5))):
        generated = engine.request(request_id).generated
        tokens = list(prompt)
        for token in generated:
            row = plain.logits(tokens)[-1]
            assert row[token] >= row.max() - 6e-3
            tokens.append(token)
    assert len(engine.request(ids[1]).generated) == 24
    assert all_pages_free(engine)
