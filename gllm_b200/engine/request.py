"""Requests and results of the Python entry point.

``GenerationRequest`` and ``GenerationResult`` keep the reference's fields,
order, defaults and meanings (gllm/engine/llm_engine_base.py:8-23).  Added:
``prompt_token_ids`` (so a tokenizer is optional), ``stop_token_ids``,
``seed`` and ``ignore_eos``.  ``RequestState`` is the scheduler's host record
(gllm/scheduler/request_state.py:7-22) plus what chunked prefill and
preemption need.
"""

from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any, NamedTuple

from gllm_b200.sampling.sampler import SamplingParams


class TokenLogProbs(NamedTuple):
    """Highest candidates of one generated token, in descending order
    (gllm/sample/logprobs.py:5-7)."""

    logprobs: list[float]
    candidate_token_ids: list[int]


@dataclass
class GenerationRequest:
    prompt: str | None = None
    max_new_tokens: int = 16
    stop_tokens: list[str] = field(default_factory=list)
    temperature: float = 0.7
    top_k: int = 40  # 0: the whole vocabulary
    top_p: float = 0.9
    max_num_logprobs: int = 0  # 0: no per-token log-probabilities
    # --- additions to the reference's request ---
    prompt_token_ids: list[int] | None = None
    stop_token_ids: list[int] = field(default_factory=list)
    seed: int = 0
    ignore_eos: bool = False


@dataclass
class GenerationResult:
    token_ids: list[int]
    logprobs: list[TokenLogProbs] | None
    text: str
    # --- additions ---
    finish_reason: str = ""          # "stop" | "length"
    token_logprobs: list[float] | None = None


class RequestStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"
    ABORTED = "aborted"


@dataclass
class RequestState:
    id: Any
    prompt_token_ids: list[int]
    max_new_tokens: int
    stop_token_ids: set[int]
    sampling: SamplingParams
    generated_token_ids: list[int] = field(default_factory=list)
    generated_logprobs: list[TokenLogProbs] = field(default_factory=list)
    generated_token_logprobs: list[float] = field(default_factory=list)
    status: RequestStatus = RequestStatus.WAITING
    # tokens (prompt + generated) whose keys and values are in the cache
    num_computed: int = 0
    num_preemptions: int = 0
    # tokens sampled on the device whose values the host has not read yet
    num_inflight: int = 0
    finish_reason: str = ""
    future: Any = None
    arrival: int = 0

    @property
    def is_finished(self) -> bool:
        return self.status in (RequestStatus.FINISHED, RequestStatus.ABORTED)

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.generated_token_ids) + self.num_inflight

    def token_slice(self, start: int, n: int) -> list[int]:
        """Tokens ``start .. start+n-1`` of prompt + generated."""
        p, end = len(self.prompt_token_ids), start + n
        known = p + len(self.generated_token_ids)
        if end > known:
            # the last token is still on the device: -1 stands for "the token last sampled for me"
            if end - known != 1 or self.num_inflight != 1:
                raise ValueError("only the very last token of a request may be in flight")
            return self.token_slice(start, n - 1) + [-1] if n > 1 else [-1]
        if end <= p:
            return self.prompt_token_ids[start:end]
        if start >= p:
            return self.generated_token_ids[start - p:end - p]
        return self.prompt_token_ids[start:] + self.generated_token_ids[:end - p]
