"""The Python entry point: ``LLMEngine``.

Same surface as the reference (gllm/engine/llm_engine.py:13-205):
``LLMEngine(hf_model, gen_params, device, local_cache_dir)``,
``generate(list[GenerationRequest]) -> list[GenerationResult]``,
``enqueue_request(req) -> asyncio.Future``, ``run()``, ``stop()``.
``hf_model`` is a model folder (config.json + safetensors, optionally
tokenizer.json); nothing is downloaded.  Underneath are this engine's own
scheduler (chunked prefill, continuous batching, preemption), step function,
cache manager, sampler and kernels.

The reference's ``run()`` cannot start (it passes ``block=`` to a function
whose parameter is ``blocking``, gllm/engine/llm_engine.py:35-38,162) and sets
each future twice (:141,178); here ``run()`` is the same loop done right:
futures are resolved once, on their own event loop's thread.
"""

from __future__ import annotations

import asyncio
import itertools
import os
import queue
from abc import ABC, abstractmethod

import torch

from gllm_b200 import ops
from gllm_b200.cache.manager import CacheManager
from gllm_b200.config.generator_params import GeneratorParams
from gllm_b200.engine.request import (
    GenerationRequest,
    GenerationResult,
    RequestState,
    TokenLogProbs,
)
from gllm_b200.engine.scheduler import ScheduledStep, Scheduler
from gllm_b200.engine.step import StepEntry, StepRunner
from gllm_b200.models.loading import load_model
from gllm_b200.sampling.sampler import Sampler, SamplingParams


class LLMEngineBase(ABC):
    """gllm/engine/llm_engine_base.py:26-30."""

    @abstractmethod
    def generate(self, reqs: list[GenerationRequest]) -> list[GenerationResult]:
        ...


class LLMEngine(LLMEngineBase):
    def __init__(
        self,
        hf_model: str,
        gen_params: GeneratorParams,
        device: str = "cuda",
        local_cache_dir: str | None = None,
    ):
        if not torch.cuda.is_available():
            raise RuntimeError("LLMEngine needs a CUDA device: this engine has no CPU path")
        if not os.path.isdir(hf_model):
            raise FileNotFoundError(
                f"{hf_model!r} is not a model folder (config.json + model.safetensors); nothing is downloaded"
            )
        dev = torch.device(device)
        if dev.type != "cuda":
            raise RuntimeError("LLMEngine runs on a CUDA device only")
        if dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        self.device = dev
        self.gen_params = gen_params
        self.alive = False
        self.config, self.model = load_model(hf_model, gen_params.model_dtype, dev)
        self.cache = CacheManager(
            self.model.cache_requirements(),
            block_size=gen_params.block_size,
            num_blocks=gen_params.resolved_num_blocks(),
            max_batch_size=gen_params.max_batch_size,
            max_seq_len=gen_params.max_seq_len,
            dtype=self.model.dtype,
            device=dev,
        )
        self.runner = StepRunner(self.model, self.cache, gen_params.max_num_batched_tokens,
                                 cuda_graphs=gen_params.cuda_graphs,
                                 prefill_graph_tokens=(gen_params.prefill_chunk,))
        self.scheduler = Scheduler(gen_params, self.cache)
        self.sampler = Sampler(dev)
        self.request_queue: queue.Queue = queue.Queue()
        self._ids = itertools.count()
        self.tokenizer = None
        tok_path = os.path.join(hf_model, "tokenizer.json")
        if os.path.isfile(tok_path):
            from tokenizers import Tokenizer

            self.tokenizer = Tokenizer.from_file(tok_path)
        self.counters = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "preemptions": 0}
        # the greedy step whose tokens the host has not read yet
        self._pending = None

    # ------------------------------------------------------------- properties
    @property
    def eos_token_ids(self) -> list[int]:
        return list(self.config.eos_token_ids)

    @property
    def max_batch_size(self) -> int:
        return self.gen_params.max_batch_size

    @property
    def max_seq_len(self) -> int:
        return self.gen_params.max_seq_len

    # -------------------------------------------------------------- tokenizer
    def tokenize(self, text: str, add_special_tokens: bool = True) -> list[int]:
        if self.tokenizer is None:
            raise RuntimeError("the model folder has no tokenizer.json: give prompt_token_ids instead of prompt")
        return self.tokenizer.encode(text, add_special_tokens=add_special_tokens).ids

    def detokenize(self, token_ids: list[int]) -> str:
        if self.tokenizer is None:
            return " ".join(str(t) for t in token_ids)
        return self.tokenizer.decode(token_ids)

    # -------------------------------------------------------------- admission
    def _make_state(self, req: GenerationRequest, future=None) -> RequestState:
        if req.prompt_token_ids is not None:
            prompt = [int(t) for t in req.prompt_token_ids]
        elif req.prompt is not None:
            prompt = self.tokenize(req.prompt)
        else:
            raise ValueError("a request needs prompt or prompt_token_ids")
        vocab = self.config.vocab_size
        if prompt and not (0 <= min(prompt) and max(prompt) < vocab):
            raise ValueError(f"a prompt token id lies outside the vocabulary of {vocab}")
        stop = set(int(t) for t in req.stop_token_ids)
        if not req.ignore_eos:
            stop |= set(self.eos_token_ids)
        for s in req.stop_tokens:
            # each stop string on its own, without special tokens
            # (the reference joins them into one string first, gllm/engine/llm_engine.py:69-71)
            stop |= set(self.tokenize(s, add_special_tokens=False))
        sampling = SamplingParams(
            temperature=req.temperature, top_k=req.top_k, top_p=req.top_p,
            max_num_logprobs=req.max_num_logprobs, seed=req.seed,
        )
        sampling.validate()
        return RequestState(
            id=next(self._ids),
            prompt_token_ids=prompt,
            max_new_tokens=req.max_new_tokens,
            stop_token_ids=stop,
            sampling=sampling,
            future=future,
        )

    def _create_result(self, state: RequestState) -> GenerationResult:
        wants_lp = state.sampling.max_num_logprobs > 0
        return GenerationResult(
            token_ids=list(state.generated_token_ids),
            logprobs=list(state.generated_logprobs) if wants_lp else None,
            text=self.detokenize(state.generated_token_ids),
            finish_reason=state.finish_reason,
            token_logprobs=list(state.generated_token_logprobs) if wants_lp else None,
        )

    # ---------------------------------------------------------------- one step
    def _resolve_pending(self) -> list[RequestState]:
        """Read the tokens of the step that is still in flight and account them."""
        if self._pending is None:
            return []
        sched, rows, slots, (host, event) = self._pending
        self._pending = None
        event.synchronize()
        values = host.tolist()
        status = values[self.runner.sampled.numel()]
        if status:
            ops.status_word(self.device).zero_()
            reasons = [text for bit, text in ops.STATUS_BITS.items() if status & bit] or [f"status {status}"]
            raise RuntimeError("a kernel reported: " + "; ".join(reasons))
        sampled = {r.id: values[slots[r.id]] for r in rows}
        return self.scheduler.resolve(sched, sampled)

    def step(self) -> list[RequestState]:
        """Schedule, run and sample one step; returns the requests that finished.

        Greedy decoding is pipelined: the sampled tokens stay on the device, where the next step
        reads them, so that step is scheduled and queued before the host has seen them; the host
        reads a step's tokens while the next one runs and may therefore report a request's end one
        call late (a request that met a stop token has then run one step too many, whose token is
        dropped).  Whenever the next schedule could depend on the tokens (somebody waits, a portion
        of a prompt runs, pages are short, sampling is not greedy) the step in flight is read first."""
        finished: list[RequestState] = []
        if self._pending is not None and not self.scheduler.can_run_ahead():
            finished += self._resolve_pending()
        sched: ScheduledStep = self.scheduler.schedule()
        self.counters["preemptions"] = self.scheduler.num_preemptions
        if not sched.entries:
            return finished + self._resolve_pending()
        entries = []
        sampling_rows = []
        for e in sched.entries:
            tokens = e.request.token_slice(e.start, e.num_tokens)
            entries.append(StepEntry(e.request.id, tokens, [e.num_tokens - 1] if e.samples else []))
            if e.samples:
                sampling_rows.append(e.request)
            if e.num_tokens == 1 and e.start > 0:
                self.counters["decode_tokens"] += 1
            else:
                self.counters["prefill_tokens"] += e.num_tokens
        all_greedy = all(r.sampling.greedy and r.sampling.max_num_logprobs == 0 for r in sampling_rows)
        logits = self.runner.run(entries, check=False, greedy=all_greedy)
        self.scheduler.advance(sched)
        self.counters["steps"] += 1
        previous, self._pending = self._pending, None
        if all_greedy:
            slots = {r.id: self.cache.requests[r.id].slot for r in sampling_rows}
            self._pending = (sched, sampling_rows, slots, self.runner.snapshot())
            if previous is not None:
                self._pending, current = previous, self._pending
                finished += self._resolve_pending()
                self._pending = current
            return finished
        if previous is not None:
            self._pending = previous
            finished += self._resolve_pending()
        sampled = {}
        if sampling_rows:
            out = self.sampler.forward(
                logits,
                [r.sampling for r in sampling_rows],
                [len(r.generated_token_ids) for r in sampling_rows],
            )
            for i, r in enumerate(sampling_rows):
                sampled[r.id] = out.token_ids[i]
                if r.sampling.max_num_logprobs > 0:
                    vals, ids = out.top_logprobs[i]
                    r.generated_logprobs.append(TokenLogProbs(vals, ids))
                    r.generated_token_logprobs.append(out.token_logprobs[i])
        ops.check_status(self.device)
        return finished + self.scheduler.resolve(sched, sampled)

    # --------------------------------------------------------------- generate
    def generate(self, reqs: list[GenerationRequest]) -> list[GenerationResult]:
        """Run ``reqs`` to completion; results in the order of ``reqs``.  More
        requests than ``max_batch_size`` are fine: the surplus waits its turn."""
        states = [self._make_state(r) for r in reqs]
        added = []
        try:
            for s in states:
                self.scheduler.add(s)
                added.append(s)
            while not all(s.is_finished for s in states):
                self.step()
                if not self.scheduler.has_work and self._pending is None:
                    break
        except BaseException:
            # a refused request, or a step that raised: nothing of this call stays queued or holds pages
            for s in added:
                self.scheduler.abort(s.id)
            if not self.scheduler.has_work:
                self._pending = None
            raise
        return [self._create_result(s) for s in states]

    def submit(self, req: GenerationRequest) -> RequestState:
        """Queue one request without running anything; ``step()`` runs it.  Returns its state
        (``id``, ``generated_token_ids``, ``is_finished``).  Raises ValueError for a request that can
        never run."""
        state = self._make_state(req)
        self.scheduler.add(state)
        return state

    def abort(self, request_id) -> bool:
        """End a waiting or running request now: its pages and its slot are free at once, a token
        of it that is still in flight is dropped.  False when no such request is live."""
        return self.scheduler.abort(request_id)

    # --------------------------------------------------- continuous batching
    def enqueue_request(self, req: GenerationRequest) -> asyncio.Future:
        """From a coroutine: returns a future of the request's GenerationResult."""
        loop = asyncio.get_running_loop()
        fut = loop.create_future()
        if not self.alive:
            fut.set_exception(RuntimeError("Engine is not running"))
            return fut
        self.request_queue.put((req, fut, loop))
        return fut

    @staticmethod
    def _resolve(fut, loop, result=None, error=None) -> None:
        def _set():
            if fut.done():
                return
            if error is not None:
                fut.set_exception(error)
            else:
                fut.set_result(result)

        loop.call_soon_threadsafe(_set)

    def _drain_queue(self, blocking: bool) -> None:
        items = []
        if blocking:
            try:
                items.append(self.request_queue.get(block=True, timeout=0.05))
            except queue.Empty:
                return
        while True:
            try:
                items.append(self.request_queue.get_nowait())
            except queue.Empty:
                break
        for req, fut, loop in items:
            try:
                state = self._make_state(req, future=(fut, loop))
                self.scheduler.add(state)
            except Exception as e:  # delivered on the request's own future
                self._resolve(fut, loop, error=e)

    def run(self) -> None:
        """The serving loop (call it on a thread of its own): admit what was
        enqueued, run a step, resolve the futures of finished requests."""
        self.alive = True
        error: BaseException | None = None
        try:
            while self.alive:
                self._drain_queue(blocking=not self.scheduler.has_work and self._pending is None)
                if not self.scheduler.has_work and self._pending is None:
                    continue
                for state in self.step():
                    if state.future is not None:
                        fut, loop = state.future
                        self._resolve(fut, loop, result=self._create_result(state))
        except BaseException as e:
            error = e
            raise
        finally:
            self.alive = False
            self._fail_outstanding(error)

    def _fail_outstanding(self, error: BaseException | None) -> None:
        """The serving loop has ended (``stop()`` or an exception): every request that is still
        queued, waiting or running gets the error on its future (nobody awaits for ever), and
        gives back its pages and its slot."""
        reason = error if isinstance(error, Exception) else RuntimeError("the engine was stopped")
        self._pending = None
        while True:
            try:
                _, fut, loop = self.request_queue.get_nowait()
            except queue.Empty:
                break
            self._resolve(fut, loop, error=reason)
        for state in list(self.scheduler.waiting) + list(self.scheduler.running):
            self.scheduler.abort(state.id)
            if state.future is not None:
                fut, loop = state.future
                self._resolve(fut, loop, error=reason)

    def stop(self) -> None:
        """Ends ``run()`` after the step it is in; requests that are not finished by then get a
        RuntimeError on their futures."""
        self.alive = False
