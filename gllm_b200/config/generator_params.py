"""Generation-time parameters chosen by the caller.

``block_size``, ``max_batch_size``, ``max_seq_len``, ``model_dtype`` and
``kv_dtype`` keep the names and meanings of the reference's dataclass
(gllm/config/generator_params.py:4-12).  Its ``cpu_offloading`` switch has no
counterpart: a B200 holds the model many times over.  The remaining fields are
this engine's own: the pool size, the per-step token budget and the largest
prompt portion, which the reference does not have because it always runs a
whole prompt in one step (gllm/llm/llm.py:204-231).
"""

from __future__ import annotations

from dataclasses import dataclass

_DTYPE_NAMES = {
    None: None,
    "bfloat16": "bfloat16",
    "bf16": "bfloat16",
    "float32": "float32",
    "fp32": "float32",
    "float": "float32",
}


@dataclass
class GeneratorParams:
    # Tokens per cache page.
    block_size: int
    # Most requests that are live (hold a state slot) at one time.
    max_batch_size: int
    # Most tokens (prompt + generated) of one request.
    max_seq_len: int
    # "bfloat16" | "float32" | None (None: what config.json names).
    model_dtype: str | None = None
    # Kept for parity; the cache holds the model dtype (no quantised caches).
    kv_dtype: str | None = None
    # Pages in each cache group's pool.  None: enough for max_batch_size
    # requests of max_seq_len tokens, the reference's sizing
    # (gllm/model/kv_cache/paged_kv_cache.py:30).
    num_blocks: int | None = None
    # Most tokens one step may run (decode tokens + prompt portions).
    max_num_batched_tokens: int = 8192
    # Largest portion of one prompt in one step.
    prefill_chunk: int = 2048
    # Capture decode-only steps in CUDA graphs (one per batch-size bucket).
    cuda_graphs: bool = True

    def __post_init__(self):
        if self.block_size <= 0 or self.max_batch_size <= 0 or self.max_seq_len <= 0:
            raise ValueError("block_size, max_batch_size and max_seq_len must be positive")
        if self.model_dtype not in _DTYPE_NAMES:
            raise ValueError(f"model_dtype must be one of bfloat16/float32, got {self.model_dtype!r}")
        if self.kv_dtype not in _DTYPE_NAMES:
            raise ValueError(f"kv_dtype must be one of bfloat16/float32, got {self.kv_dtype!r}")
        self.model_dtype = _DTYPE_NAMES[self.model_dtype]
        self.kv_dtype = _DTYPE_NAMES[self.kv_dtype]
        if self.kv_dtype is not None and self.model_dtype is not None and self.kv_dtype != self.model_dtype:
            raise ValueError(
                "kv_dtype differs from model_dtype: the cache always holds the model's dtype "
                "(reduced-precision caches are not part of this engine)"
            )
        if self.max_num_batched_tokens <= 0 or self.prefill_chunk <= 0:
            raise ValueError("max_num_batched_tokens and prefill_chunk must be positive")
        if self.num_blocks is not None and self.num_blocks <= 0:
            raise ValueError("num_blocks must be positive")

    @property
    def max_blocks_per_request(self) -> int:
        return -(-self.max_seq_len // self.block_size)

    def resolved_num_blocks(self) -> int:
        if self.num_blocks is not None:
            return self.num_blocks
        return self.max_batch_size * self.max_blocks_per_request
