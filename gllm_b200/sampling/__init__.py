"""Sampling: per-request parameters and the sampler that turns logits into tokens."""

from gllm_b200.sampling.sampler import Sampler, SamplerOutput, SamplingParams

__all__ = ["Sampler", "SamplerOutput", "SamplingParams"]
