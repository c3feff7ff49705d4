"""The scheduler: which requests run in the next step, and how many tokens each.

The reference has no scheduler beyond admission: every queued request joins the
next step with its whole prompt, a full batch *rejects* newcomers, and the page
pool is sized so it cannot run short; when it does, the engine crashes
(gllm/engine/llm_engine.py:55-113,156-180, gllm/model/kv_cache/paged_kv_cache.py:81-97).

Here, per step, under a token budget (``max_num_batched_tokens``):
  1. every running request that is decoding gets its one token;
  2. running requests still in their prompt get a portion
     (<= ``prefill_chunk``, <= budget left);
  3. waiting requests are admitted first-come first-served while a state slot,
     budget and pages are there: pages for the first portion now, and, beside
     what the running requests still need for the rest of THEIR prompts, pages
     for the rest of this one (so a prompt that is admitted can be finished;
     without this reservation long prompts over a small pool were admitted on
     their first portion, preempted on a later one and recomputed, again and
     again).  A full engine leaves requests waiting; only impossible requests
     are refused at ``add``.
When pages run out while a running request needs one more, the most recently
admitted running request is preempted: its pages and slot are given back at
once, it returns to the head of the waiting queue and later recomputes its
prompt and the tokens it had generated (counted in ``num_preemptions``).
Finishing frees pages and slot at once.  This file does no device work.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from gllm_b200.cache.manager import CacheManager
from gllm_b200.config.generator_params import GeneratorParams
from gllm_b200.engine.request import RequestState, RequestStatus


@dataclass
class ScheduledEntry:
    request: RequestState
    start: int           # first token (index into prompt + generated) of the portion
    num_tokens: int
    samples: bool        # the portion ends at the request's last token: sample from it


@dataclass
class ScheduledStep:
    entries: list[ScheduledEntry] = field(default_factory=list)
    preempted: list[RequestState] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(e.num_tokens for e in self.entries)


class Scheduler:
    def __init__(self, params: GeneratorParams, cache: CacheManager):
        self.params = params
        self.cache = cache
        self.waiting: deque[RequestState] = deque()
        self.running: list[RequestState] = []
        self._arrivals = 0
        self.num_preemptions = 0
        self.num_steps = 0

    # ------------------------------------------------------------- admission
    def add(self, req: RequestState) -> None:
        """Queue a request.  Raises ValueError for one that can never run, with
        the reference's conditions (gllm/engine/llm_engine.py:73-82) plus the
        pool size."""
        n_prompt = len(req.prompt_token_ids)
        if n_prompt == 0:
            raise ValueError("the prompt has no tokens")
        allowed = self.params.max_seq_len - n_prompt
        if allowed <= 0:
            raise ValueError(
                f"Prompt has {n_prompt} tokens, but the engine only supports {self.params.max_seq_len}."
            )
        if req.max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be > 0.")
        req.max_new_tokens = min(allowed, req.max_new_tokens)
        worst = n_prompt + req.max_new_tokens
        worst_pages = max(self.cache.pages_for_admission(worst).values(), default=0)
        if worst_pages > self.cache.num_blocks:
            raise ValueError(
                f"the request may grow to {worst} tokens = {worst_pages} pages, the pool has {self.cache.num_blocks}"
            )
        req.status = RequestStatus.WAITING
        req.arrival = self._arrivals
        self._arrivals += 1
        self.waiting.append(req)

    def abort(self, request_id) -> bool:
        for req in list(self.waiting):
            if req.id == request_id:
                self.waiting.remove(req)
                req.status = RequestStatus.ABORTED
                return True
        for req in self.running:
            if req.id == request_id:
                self._release(req)
                self.running.remove(req)
                req.status = RequestStatus.ABORTED
                return True
        return False

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # -------------------------------------------------------------- one step
    def _release(self, req: RequestState) -> None:
        if req.id in self.cache.requests:
            self.cache.free_request(req.id)

    def _preempt(self, victim: RequestState, step: ScheduledStep) -> None:
        self._release(victim)
        self.running.remove(victim)
        victim.status = RequestStatus.WAITING
        victim.num_computed = 0
        victim.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(victim)
        step.preempted.append(victim)
        step.entries = [e for e in step.entries if e.request is not victim]

    def schedule(self) -> ScheduledStep:
        step = ScheduledStep()
        budget = self.params.max_num_batched_tokens
        groups = [g.index for g in self.cache.groups]
        # pages promised to this step's entries, per entry and in total
        promised: dict[int, dict[int, int]] = {}
        taken = {g: 0 for g in groups}
        new_slots = 0

        def fits(need: dict[int, int]) -> bool:
            return all(self.cache.groups[g].allocator.num_free - taken[g] >= n for g, n in need.items())

        def promise(req, need) -> None:
            promised[id(req)] = need
            for g, n in need.items():
                taken[g] += n

        # 1 + 2: running requests, decoding ones first, each in admission order
        order = [r for r in self.running if r.num_tokens - r.num_computed == 1] + [
            r for r in self.running if r.num_tokens - r.num_computed > 1
        ]
        for req in order:
            if req.status is not RequestStatus.RUNNING:
                continue  # preempted a moment ago
            if len(req.generated_token_ids) + req.num_inflight >= req.max_new_tokens:
                continue  # its last token is in flight: nothing more to run
            pending = req.num_tokens - req.num_computed
            n = min(pending, self.params.prefill_chunk, budget)
            if n <= 0:
                continue
            while True:
                need = self.cache.pages_needed(req.id, n)
                if fits(need):
                    promise(req, need)
                    step.entries.append(
                        ScheduledEntry(req, req.num_computed, n, req.num_computed + n == req.num_tokens)
                    )
                    budget -= n
                    break
                # out of pages: the most recently admitted running request gives way
                victim = self.running[-1]
                for e in step.entries:
                    if e.request is victim:
                        budget += e.num_tokens
                        for g, k in promised.pop(id(victim)).items():
                            taken[g] -= k
                self._preempt(victim, step)
                if victim is req:
                    break
        # pages the running requests will still ask for to hold the tokens they are known to have
        # (the rest of their prompts), beyond what they hold and what this step promised them
        reserved = {g: 0 for g in groups}
        for req in self.running:
            if req.id in self.cache.requests:
                rest = self.cache.pages_needed(req.id, req.num_tokens - self.cache.requests[req.id].num_tokens)
            else:
                rest = self.cache.pages_for_admission(req.num_tokens)
            for g, n in rest.items():
                reserved[g] += max(0, n - promised.get(id(req), {}).get(g, 0))
        # 3: admissions, first come first served
        while self.waiting and budget > 0 and len(self.running) < self.params.max_batch_size:
            req = self.waiting[0]
            if any(req is v for v in step.preempted):
                break  # not in the step that preempted it
            if self.cache.slots.num_free - new_slots <= 0:
                break
            n = min(req.num_tokens, self.params.prefill_chunk, budget)
            need = self.cache.pages_for_admission(n)
            if not fits(need):
                break
            whole = self.cache.pages_for_admission(req.num_tokens)
            if self.running and not all(
                    self.cache.groups[g].allocator.num_free - taken[g] - reserved[g] >= whole[g] for g in groups):
                break  # its whole prompt would not fit beside what the running prompts still need
            for g in groups:
                reserved[g] += whole[g] - need[g]
            promise(req, need)
            new_slots += 1
            self.waiting.popleft()
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            step.entries.append(ScheduledEntry(req, 0, n, n == req.num_tokens))
            budget -= n
        self.num_steps += 1
        return step

    # ------------------------------------------------------------ after a step
    def can_run_ahead(self) -> bool:
        """True when the next step can be scheduled before the previous step's tokens are known:
        nobody waits, everybody decodes, and every request finds room for one more token, so the
        schedule holds no admission and no preemption."""
        if self.waiting or not self.running:
            return False
        need = {g.index: 0 for g in self.cache.groups}
        for req in self.running:
            if req.num_tokens - req.num_computed != 1 or req.id not in self.cache.requests:
                return False
            for g, n in self.cache.pages_needed(req.id, 1).items():
                need[g] += n
        return all(self.cache.groups[g].allocator.num_free >= n for g, n in need.items())

    def advance(self, step: ScheduledStep) -> None:
        """The step has been queued on the device: count its tokens as computed and the tokens
        it will sample as in flight."""
        for e in step.entries:
            e.request.num_computed += e.num_tokens
            if e.samples:
                e.request.num_inflight += 1

    def resolve(self, step: ScheduledStep, sampled: dict) -> list[RequestState]:
        """The host has read the step's tokens: ``sampled[request.id]`` for every entry that
        sampled.  Returns the requests that finished; their pages and slots are already free.
        A request that ended meanwhile (a stop token one step earlier, an abort) ignores its token."""
        finished = []
        for e in step.entries:
            req = e.request
            if not e.samples:
                continue
            req.num_inflight -= 1
            if req.status is not RequestStatus.RUNNING:
                continue
            token = sampled[req.id]
            req.generated_token_ids.append(token)
            # gllm/engine/llm_engine.py:126-127: stop token (kept in the output) or length
            if token in req.stop_token_ids:
                req.finish_reason = "stop"
            elif len(req.generated_token_ids) >= req.max_new_tokens:
                req.finish_reason = "length"
            if req.finish_reason:
                req.status = RequestStatus.FINISHED
                self._release(req)
                self.running.remove(req)
                finished.append(req)
        return finished

    def update(self, step: ScheduledStep, sampled: dict) -> list[RequestState]:
        """``advance`` and ``resolve`` in one go (the step's tokens are known already)."""
        self.advance(step)
        return self.resolve(step, sampled)
