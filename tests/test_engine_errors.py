"""The engine's error paths, on the host: a step that raises ends ``run()`` with
every outstanding future resolved, ``stop()`` does the same, and a ``generate()``
call that is refused half-way leaves nothing queued.  The engine object is put
together without a device: its scheduler and cache manager are the real ones,
its step function is a stand-in."""

import asyncio
import itertools
import queue
import threading
import time
import types

import pytest
import torch

from gllm_b200.cache import CacheManager
from gllm_b200.config import GeneratorParams
from gllm_b200.engine.llm_engine import LLMEngine
from gllm_b200.engine.request import GenerationRequest
from gllm_b200.engine.scheduler import Scheduler
from gllm_b200.parts.base import KVPageRequirement


def host_engine(step):
    params = GeneratorParams(block_size=4, max_batch_size=4, max_seq_len=32, num_blocks=16,
                             max_num_batched_tokens=16, prefill_chunk=8)
    cache = CacheManager([(KVPageRequirement.keys_and_values(1, 16), None, None)], 4, 16, 4, 32, torch.float32, "cpu",
                         allocate_pools=False)
    eng = object.__new__(LLMEngine)
    eng.gen_params = params
    eng.cache = cache
    eng.scheduler = Scheduler(params, cache)
    eng.config = types.SimpleNamespace(vocab_size=100, eos_token_ids=(99,))
    eng.request_queue = queue.Queue()
    eng._ids = itertools.count()
    eng.tokenizer = None
    eng._pending = None
    eng.alive = False
    eng.step = types.MethodType(step, eng)
    return eng


def take_pages_then_raise(eng):
    """A step that admits what waits (pages and slots are taken) and then fails."""
    sched = eng.scheduler.schedule()
    for e in sched.entries:
        if e.request.id not in eng.cache.requests:
            eng.cache.add_request(e.request.id)
        eng.cache.append(e.request.id, e.num_tokens)
        eng.cache.commit(e.request.id, e.num_tokens)
    raise RuntimeError("a kernel reported: test failure")


def never_finishes(eng):
    """A slow step that samples token 1 for everybody (29 steps of 5 ms before a request's length ends it)."""
    sched = eng.scheduler.schedule()
    for e in sched.entries:
        if e.request.id not in eng.cache.requests:
            eng.cache.add_request(e.request.id)
        eng.cache.append(e.request.id, e.num_tokens)
        eng.cache.commit(e.request.id, e.num_tokens)
    time.sleep(0.005)
    return eng.scheduler.update(sched, {e.request.id: 1 for e in sched.entries if e.samples})


def serve(eng, coro_factory):
    """Run ``eng.run()`` on a thread and the coroutine on an event loop; returns (results, thread error)."""
    errors = []

    def loop_body():
        try:
            eng.run()
        except BaseException as e:      # noqa: BLE001
            errors.append(e)

    async def main():
        t = threading.Thread(target=loop_body, daemon=True)
        t.start()
        while not eng.alive and t.is_alive():
            await asyncio.sleep(0.001)
        out = await coro_factory()
        t.join(timeout=5)
        assert not t.is_alive()
        return out

    return asyncio.run(asyncio.wait_for(main(), timeout=20)), errors


def test_a_step_that_raises_resolves_every_future_and_frees_everything():
    eng = host_engine(take_pages_then_raise)

    async def clients():
        futs = [eng.enqueue_request(GenerationRequest(prompt_token_ids=[1, 2, 3, 4, 5], max_new_tokens=4))
                for _ in range(6)]                      # more than max_batch_size: some still wait
        return await asyncio.gather(*futs, return_exceptions=True)

    results, errors = serve(eng, clients)
    assert len(results) == 6 and all(isinstance(r, RuntimeError) for r in results)
    assert "test failure" in str(results[0])
    assert errors and "test failure" in str(errors[0])
    assert not eng.alive and not eng.scheduler.has_work and not eng.cache.requests
    assert eng.cache.num_free_pages() == 16 and eng.cache.slots.num_free == 4
    eng.cache.check_invariants()


def test_stop_with_work_outstanding_resolves_the_futures():
    eng = host_engine(never_finishes)

    async def clients():
        futs = [eng.enqueue_request(GenerationRequest(prompt_token_ids=[1, 2, 3], max_new_tokens=1000,
                                                      ignore_eos=True)) for _ in range(3)]
        await asyncio.sleep(0.05)
        eng.stop()
        return await asyncio.gather(*futs, return_exceptions=True)

    results, errors = serve(eng, clients)
    assert not errors
    assert all(isinstance(r, RuntimeError) and "stopped" in str(r) for r in results)
    assert not eng.scheduler.has_work and eng.cache.num_free_pages() == 16


def test_a_refused_request_leaves_nothing_of_its_generate_call_queued():
    eng = host_engine(never_finishes)
    good = GenerationRequest(prompt_token_ids=[1, 2, 3], max_new_tokens=2)
    too_long = GenerationRequest(prompt_token_ids=list(range(40)), max_new_tokens=2)     # > max_seq_len
    with pytest.raises(ValueError):
        eng.generate([good, good, too_long])
    assert not eng.scheduler.has_work and not eng.cache.requests


def test_submit_and_abort_are_public():
    eng = host_engine(never_finishes)
    st = eng.submit(GenerationRequest(prompt_token_ids=[1, 2, 3], max_new_tokens=2))
    eng.step()
    assert st.id in eng.cache.requests
    assert eng.abort(st.id) and not eng.cache.requests and not eng.abort(st.id)
