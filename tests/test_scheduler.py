"""The scheduler's decisions, on the host with a pretend model that samples
token 1 for everybody: admission, portions under the token budget, decoding,
finishing and freeing, and what happens when pages run out."""

import pytest
import torch

from gllm_b200.cache import CacheManager
from gllm_b200.config import GeneratorParams
from gllm_b200.engine.request import RequestState, RequestStatus
from gllm_b200.engine.scheduler import Scheduler
from gllm_b200.parts.base import KVPageRequirement
from gllm_b200.sampling import SamplingParams


def setup(block_size=4, max_batch=4, max_seq_len=64, num_blocks=32, budget=16, chunk=8):
    params = GeneratorParams(block_size=block_size, max_batch_size=max_batch, max_seq_len=max_seq_len,
                             num_blocks=num_blocks, max_num_batched_tokens=budget, prefill_chunk=chunk)
    cache = CacheManager([(KVPageRequirement.keys_and_values(1, 16), None, None)], block_size, num_blocks, max_batch, max_seq_len,
                         torch.float32, "cpu", allocate_pools=False)
    return params, cache, Scheduler(params, cache)


def request(rid, n_prompt, max_new=4, stop=()):
    return RequestState(id=rid, prompt_token_ids=list(range(10, 10 + n_prompt)), max_new_tokens=max_new,
                        stop_token_ids=set(stop), sampling=SamplingParams())


def run_step(sched, cache, token=1):
    """What the engine does around a step, without a model."""
    step = sched.schedule()
    for e in step.entries:
        if e.request.id not in cache.requests:
            cache.add_request(e.request.id)
        assert e.start == cache.requests[e.request.id].num_tokens      # portions run in order
        cache.append(e.request.id, e.num_tokens)                       # must succeed: the scheduler promised
        cache.commit(e.request.id, e.num_tokens)
    finished = sched.update(step, {e.request.id: token for e in step.entries if e.samples})
    cache.check_invariants()
    return step, finished


def test_portions_under_budget_then_decode_then_finish():
    params, cache, sched = setup(budget=16, chunk=8)
    a, b = request("a", 20, max_new=3), request("b", 5, max_new=2)
    sched.add(a)
    sched.add(b)
    s1, _ = run_step(sched, cache)
    assert [(e.request.id, e.start, e.num_tokens, e.samples) for e in s1.entries] == [("a", 0, 8, False), ("b", 0, 5, True)]
    s2, _ = run_step(sched, cache)          # b decodes first (one token), a gets its next portion
    assert [(e.request.id, e.start, e.num_tokens, e.samples) for e in s2.entries] == [("b", 5, 1, True), ("a", 8, 8, False)]
    assert b.status is RequestStatus.FINISHED and b.finish_reason == "length" and "b" not in cache.requests
    s3, _ = run_step(sched, cache)
    assert [(e.request.id, e.start, e.num_tokens, e.samples) for e in s3.entries] == [("a", 16, 4, True)]
    for _ in range(2):
        run_step(sched, cache)
    assert a.is_finished and a.generated_token_ids == [1, 1, 1] and not sched.has_work
    assert cache.num_free_pages() == 32 and cache.slots.num_free == 4


def test_token_budget_is_never_exceeded_and_a_full_engine_leaves_requests_waiting():
    params, cache, sched = setup(max_batch=2, budget=10, chunk=6)
    reqs = [request(i, 9, max_new=5) for i in range(5)]
    for r in reqs:
        sched.add(r)
    seen_running = 0
    while sched.has_work:
        step, _ = run_step(sched, cache)
        assert 0 < step.num_tokens <= 10
        assert all(e.num_tokens <= 6 for e in step.entries)
        assert len(sched.running) <= 2
        seen_running = max(seen_running, len(sched.running))
    assert seen_running == 2 and all(r.is_finished and len(r.generated_token_ids) == 5 for r in reqs)
    # first come, first served
    assert [r.id for r in sorted(reqs, key=lambda r: r.arrival)] == [0, 1, 2, 3, 4]


def test_stop_token_ends_a_request_and_stays_in_the_output():
    params, cache, sched = setup()
    r = request("a", 3, max_new=10, stop=(1,))
    sched.add(r)
    run_step(sched, cache, token=1)
    assert r.is_finished and r.finish_reason == "stop" and r.generated_token_ids == [1]


def test_impossible_requests_are_refused_with_the_reference_conditions():
    params, cache, sched = setup(max_seq_len=16, num_blocks=3)
    with pytest.raises(ValueError, match="only supports 16"):
        sched.add(request("long", 16))
    with pytest.raises(ValueError, match="max_new_tokens"):
        sched.add(request("zero", 4, max_new=0))
    with pytest.raises(ValueError, match="pages"):
        sched.add(request("big", 10, max_new=6))          # 16 tokens = 4 pages > pool of 3
    r = request("clamped", 10, max_new=100)
    params2, cache2, sched2 = setup(max_seq_len=16, num_blocks=8)
    sched2.add(r)
    assert r.max_new_tokens == 6                           # clamped to max_seq_len - prompt


def test_out_of_pages_preempts_the_newest_and_recomputes_it():
    # 6 pages of 4 tokens; two requests of 8 prompt tokens fill 4 pages, then both grow
    params, cache, sched = setup(num_blocks=6, budget=32, chunk=32, max_seq_len=24)
    old, new = request("old", 8, max_new=12), request("new", 8, max_new=12)
    sched.add(old)
    sched.add(new)
    preempted_at = None
    steps = 0
    while sched.has_work:
        step, _ = run_step(sched, cache)
        steps += 1
        if step.preempted and preempted_at is None:
            preempted_at = steps
            assert [r.id for r in step.preempted] == ["new"]          # the most recently admitted gives way
            assert "new" not in cache.requests and new.status is RequestStatus.WAITING
            assert new.num_computed == 0 and new.generated_token_ids  # keeps what it generated
            assert all(e.request is old for e in step.entries)        # not re-admitted in the same step
        assert steps < 200
    assert preempted_at is not None and sched.num_preemptions >= 1
    assert old.is_finished and new.is_finished
    assert len(old.generated_token_ids) == 12 and len(new.generated_token_ids) == 12
    assert cache.num_free_pages() == 6


def test_recompute_after_preemption_covers_prompt_and_generated_tokens():
    params, cache, sched = setup(num_blocks=6, budget=32, chunk=32, max_seq_len=24)
    old, new = request("old", 8, max_new=12), request("new", 8, max_new=12)
    sched.add(old)
    sched.add(new)
    checked = False
    while sched.has_work:
        before = new.num_tokens
        step, _ = run_step(sched, cache)
        for e in step.entries:
            if e.request is new and new.num_preemptions and e.start == 0:
                # the portion after a preemption restarts at 0 and runs over prompt + generated so far
                assert e.num_tokens == before and e.samples
                assert new.token_slice(0, e.num_tokens) == new.prompt_token_ids + new.generated_token_ids[:before - 8]
                checked = True
    assert checked


def test_abort_frees_at_once():
    params, cache, sched = setup()
    a, b = request("a", 6), request("b", 6)
    sched.add(a)
    sched.add(b)
    run_step(sched, cache)
    assert sched.abort("a") and a.status is RequestStatus.ABORTED and "a" not in cache.requests
    assert not sched.abort("nobody")
    while sched.has_work:
        run_step(sched, cache)
    assert b.is_finished and cache.num_free_pages() == 32


def test_token_slice():
    r = request("a", 5)
    r.generated_token_ids = [100, 101, 102]
    assert r.token_slice(0, 5) == [10, 11, 12, 13, 14]
    assert r.token_slice(3, 4) == [13, 14, 100, 101]
    assert r.token_slice(6, 2) == [101, 102]
    assert r.token_slice(7, 1) == [102]


def test_running_ahead_reads_tokens_one_step_late():
    """Greedy decoding is pipelined: a step is scheduled while the tokens of the step before are
    still on the device.  Length limits are honoured exactly; a stop token is seen one step late
    and the token of the step too many is dropped."""
    params, cache, sched = setup(num_blocks=32, budget=64, chunk=64)
    a, b = request("a", 6, max_new=3), request("b", 4, max_new=10, stop=(7,))
    sched.add(a)
    sched.add(b)
    assert not sched.can_run_ahead()                      # somebody waits
    pending = None
    tokens_for = {"a": iter([5, 5, 5, 5, 5]), "b": iter([1, 7, 9, 9, 9])}   # b meets its stop token second
    steps = 0
    while sched.has_work:
        if pending is not None and not sched.can_run_ahead():
            sched.resolve(*pending)
            pending = None
        step = sched.schedule()
        if not step.entries:
            if pending is not None:
                sched.resolve(*pending)
                pending = None
            continue
        for e in step.entries:
            if e.request.id not in cache.requests:
                cache.add_request(e.request.id)
            toks = e.request.token_slice(e.start, e.num_tokens)
            assert len(toks) == e.num_tokens
            if e.start >= 6 or (e.request is b and e.start >= 4):
                assert toks == [-1] or e.request.num_inflight == 0   # the device supplies the token in flight
            cache.append(e.request.id, e.num_tokens)
            cache.commit(e.request.id, e.num_tokens)
        sched.advance(step)
        sampled = {e.request.id: next(tokens_for[e.request.id]) for e in step.entries if e.samples}
        previous, pending = pending, (step, sampled)
        if previous is not None:
            sched.resolve(*previous)
        steps += 1
        assert steps < 50
    if pending is not None:
        sched.resolve(*pending)
    assert a.generated_token_ids == [5, 5, 5] and a.finish_reason == "length"       # never a fourth step for a
    assert b.generated_token_ids == [1, 7] and b.finish_reason == "stop"            # the 9 of the extra step is dropped
    assert a.num_inflight == 0 and b.num_inflight == 0
    assert cache.num_free_pages() == 32 and cache.slots.num_free == 4
    cache.check_invariants()


def test_a_prompt_is_admitted_only_when_all_of_it_fits_beside_the_running_prompts():
    # 10 pages of 4 tokens, portions of 8 tokens: three prompts of 24 tokens (6 pages each).  Admitted on their
    # first portion alone, the second would take pages the first still needs and one of them would be preempted
    # and recomputed; with the reservation the second waits until the first has finished, and nothing is preempted.
    params, cache, sched = setup(num_blocks=10, budget=16, chunk=8, max_seq_len=40, max_batch=4)
    reqs = [request(f"r{i}", 24, max_new=2) for i in range(3)]
    for r in reqs:
        sched.add(r)
    steps = 0
    most_running = 0
    while sched.has_work:
        step, _ = run_step(sched, cache)
        most_running = max(most_running, len(sched.running))
        assert not step.preempted
        steps += 1
        assert steps < 100
    assert sched.num_preemptions == 0 and all(r.is_finished for r in reqs)
    assert most_running == 1                       # 6 + 6 pages never fit the 10
    # short prompts still share the engine: four of 8 tokens (2 pages each, 3 with their generated tokens)
    params, cache, sched = setup(num_blocks=12, budget=32, chunk=8, max_seq_len=16, max_batch=4)
    for i in range(4):
        sched.add(request(f"s{i}", 8, max_new=3))
    run_step(sched, cache)
    assert len(sched.running) == 4
