"""The sampler: logits of a step's wanted rows in, one token per row out.

Options keep the reference's names, defaults and meanings
(gllm/engine/llm_engine_base.py:9-16, gllm/sample/sampler.py:67-107):
``temperature`` 0.7, ``top_k`` 40 (0 = whole vocabulary), ``top_p`` 0.9,
``max_num_logprobs`` 0.  The reference draws with the global torch generator;
here every request has a ``seed`` and each of its tokens uses the counter of
that token, so a request's samples do not depend on its neighbours.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from gllm_b200 import ops


@dataclass
class SamplingParams:
    temperature: float = 0.7
    top_k: int = 40          # 0: whole vocabulary; 1: greedy
    top_p: float = 0.9
    max_num_logprobs: int = 0
    seed: int = 0

    def validate(self) -> None:
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0 (0 is greedy)")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0 (0 is the whole vocabulary)")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")
        if not 0 <= self.max_num_logprobs <= ops.MAX_LOGPROBS:
            raise ValueError(f"max_num_logprobs must be between 0 and {ops.MAX_LOGPROBS}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0 or self.top_k == 1


@dataclass
class SamplerOutput:
    token_ids: list[int]
    # log-probability of each sampled token (log_softmax of the raw logits)
    token_logprobs: list[float]
    # per row (values, ids) of the highest candidates in descending order, as
    # the reference returns them (gllm/sample/sampler.py:90-106); None if not asked
    top_logprobs: list[tuple[list[float], list[int]] | None]


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)

    def sample_greedy_device(self, logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Argmax of every row on the device (no host sync)."""
        return ops.argmax(logits, out)

    def forward(self, logits: torch.Tensor, params: list[SamplingParams], counters: list[int]) -> SamplerOutput:
        rows = logits.shape[0]
        if rows != len(params) or rows != len(counters):
            raise ValueError("one SamplingParams and one counter per row")
        if all(p.greedy and p.max_num_logprobs == 0 for p in params):
            tokens = ops.argmax(logits).tolist()
            return SamplerOutput(tokens, [float("nan")] * rows, [None] * rows)
        host = np.empty((rows, 6), dtype=np.float64)
        for i, (p, c) in enumerate(zip(params, counters)):
            host[i] = (p.temperature, p.top_k, p.top_p, p.seed, c, p.max_num_logprobs)
        dev = self.device
        t = torch.from_numpy(host)
        max_lp = max(p.max_num_logprobs for p in params)
        out = ops.sample(
            logits,
            t[:, 0].to(torch.float32).to(dev),
            t[:, 1].to(torch.int32).to(dev),
            t[:, 2].to(torch.float32).to(dev),
            torch.tensor([p.seed for p in params], dtype=torch.int64, device=dev),
            t[:, 4].to(torch.int32).to(dev),
            t[:, 5].to(torch.int32).to(dev) if max_lp else None,
            max_logprobs=max_lp,
        )
        tokens = out["tokens"].tolist()
        token_lp = out["logprobs"].tolist()
        tops: list = [None] * rows
        if max_lp:
            ncand = out["num_candidates"].tolist()
            vals, ids = out["top_logprobs"].tolist(), out["top_ids"].tolist()
            for i, p in enumerate(params):
                if p.max_num_logprobs:
                    n = min(p.max_num_logprobs, ncand[i])
                    tops[i] = (vals[i][:n], ids[i][:n])
        return SamplerOutput(tokens, token_lp, tops)
