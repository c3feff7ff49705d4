"""Tensor-core attention kernels of the bf16 path (prefill tiles and split-KV
decode) over the paged cache."""

from __future__ import annotations


def supports(head_dim: int, block_size: int) -> bool:
    return False


def paged_attention_bf16(*args, **kwargs):
    raise NotImplementedError
