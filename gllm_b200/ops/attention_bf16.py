"""Attention kernels of the bf16 path over the paged cache: split-KV decode
for requests that bring one token, tiled prefill for the rest.

The step function lays the flat batch out with all multi-token portions first
and the single decoded tokens after them (``StepContext.num_prefill_tokens``),
so each kernel works on one contiguous run of tokens.
"""

from __future__ import annotations

import os
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from gllm_b200.ops.build import load_module

P = c_void_p
_DECODE_HEAD_DIMS = (32, 64, 128)

_PREFILL_HEAD_DIMS = (32, 64, 128)
_decode = None
_prefill = None


def _prefill_fn():
    global _prefill
    if _prefill is None:
        lib = load_module("attention_prefill_bf16")
        f = lib.gllm_attention_prefill_bf16
        f.argtypes = [P, c_int64, P, c_int64, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                      c_float, c_int, P, P]
        f.restype = c_int
        _prefill = f
    return _prefill


_prefill_tmem = None
# portions shorter than this run the mma.sync kernel (its 64-row tiles waste less on short portions)
TMEM_MIN_Q_LEN = 32


def _prefill_tmem_fn():
    global _prefill_tmem
    if _prefill_tmem is None:
        lib = load_module("attention_prefill_tmem")
        f = lib.gllm_attention_prefill_tmem
        f.argtypes = [P, c_int64, P, c_int64, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                      c_int, c_float, c_int, P, P]
        f.restype = c_int
        lib.gllm_attention_prefill_tmem_supports.argtypes = [c_int, c_int]
        lib.gllm_attention_prefill_tmem_supports.restype = c_int
        _prefill_tmem = (f, lib.gllm_attention_prefill_tmem_supports)
    return _prefill_tmem


def prefill_tmem_supports(head_dim: int, block_size: int, q: torch.Tensor, cache_layer: torch.Tensor) -> bool:
    return (head_dim in (64, 128) and bool(_prefill_tmem_fn()[1](head_dim, block_size))
            and q.data_ptr() % 16 == 0 and cache_layer.data_ptr() % 16 == 0 and q.stride(0) % 8 == 0)


def prefill_attention_tmem(q, q_stride, cache_layer, block_table, cu_q, ctx_lens, slots, num_requests, max_q_len,
                           num_heads, scale, window, out):
    """tcgen05 attention of the first ``num_requests`` requests of the flat batch."""
    from gllm_b200 import ops

    num_pages, _, hkv, block_size, d = cache_layer.shape
    code = _prefill_tmem_fn()[0](
        q.data_ptr(), q_stride, out.data_ptr(), out.stride(0), cache_layer.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), cu_q.data_ptr(), ctx_lens.data_ptr(), slots.data_ptr(), num_requests, max_q_len,
        q.shape[0], num_heads, hkv, d, block_size, num_pages, float(scale), int(window),
        ops.status_word(q.device).data_ptr(), ops._stream(),
    )
    ops._check(code, "attention_prefill_tmem")
    return out


def prefill_supports(head_dim: int, block_size: int) -> bool:
    return head_dim in _PREFILL_HEAD_DIMS and (block_size * head_dim) % 8 == 0


def prefill_attention(q, q_stride, cache_layer, block_table, cu_q, ctx_lens, slots, num_requests, max_q_len,
                      num_heads, scale, window, out):
    """Tensor-core attention of the first ``num_requests`` requests of the
    flat batch (portions of prompts)."""
    from gllm_b200 import ops

    num_pages, _, hkv, block_size, d = cache_layer.shape
    code = _prefill_fn()(
        q.data_ptr(), q_stride, out.data_ptr(), out.stride(0), cache_layer.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), cu_q.data_ptr(), ctx_lens.data_ptr(), slots.data_ptr(), num_requests, max_q_len,
        num_heads, hkv, d, block_size, num_pages, float(scale), int(window),
        ops.status_word(q.device).data_ptr(), ops._stream(),
    )
    ops._check(code, "attention_prefill_bf16")
    return out


def _decode_fn():
    global _decode
    if _decode is None:
        lib = load_module("attention_bf16")
        f = lib.gllm_attention_decode_bf16
        f.argtypes = [P, c_int64, P, c_int64, P, P, c_int, P, P, c_int, P, P, c_int, c_int, c_int, c_int, c_int,
                      c_int, c_float, c_int, P, P]
        f.restype = c_int
        lib.gllm_attention_decode_chunk.argtypes = [c_int]
        lib.gllm_attention_decode_chunk.restype = c_int
        _decode = (f, lib.gllm_attention_decode_chunk)
    return _decode


_decode_stream = None
STREAM_SPAN = 128
# the stream kernel has one work item per 128 keys of a request: below this many items the split
# kernel, with a work item per kv head as well, fills the machine better
# (GLLM_B200_STREAM_MIN_ITEMS overrides the threshold: tests use 1 to run small steps through it)
STREAM_MIN_ITEMS = int(os.environ.get("GLLM_B200_STREAM_MIN_ITEMS", 296))


def _decode_stream_fn():
    global _decode_stream
    if _decode_stream is None:
        lib = load_module("attention_decode_tma")
        f = lib.gllm_attention_decode_stream
        f.argtypes = [P, c_int64, P, c_int64, P, P, c_int, P, P, c_int, P, P, c_int, c_int, c_int, c_int, c_int,
                      c_int, c_float, c_int, P, P]
        f.restype = c_int
        lib.gllm_attention_decode_stream_parts.argtypes = [c_int, c_int, c_int, c_int]
        lib.gllm_attention_decode_stream_parts.restype = c_int
        _decode_stream = (f, lib.gllm_attention_decode_stream_parts)
    return _decode_stream


def decode_stream_parts(head_dim: int, num_heads: int, num_kv_heads: int, block_size: int,
                        q: torch.Tensor, cache_layer: torch.Tensor) -> int:
    """Partial results per 128 keys that the persistent TMA kernel leaves for these sizes; 0 when it
    does not take them (head sizes 64 and 128, up to 8 kv heads of up to 16 query heads, pages of 16
    or 32 tokens, 16-byte aligned operands)."""
    if head_dim not in (64, 128) or q.data_ptr() % 16 or cache_layer.data_ptr() % 16 or q.stride(0) % 8:
        return 0
    return int(_decode_stream_fn()[1](head_dim, num_heads, num_kv_heads, block_size))


def decode_chunk(head_dim: int) -> int:
    """Keys per split of the decode kernel for this head size: a constant, so
    the cut of a request's keys depends on positions only."""
    return _decode_fn()[1](head_dim)


def supports(head_dim: int, block_size: int) -> bool:
    return head_dim in _DECODE_HEAD_DIMS and (block_size * head_dim) % 8 == 0


def decode_scratch_elems(num_queries: int, num_heads: int, head_dim: int, max_seq_len: int) -> tuple[int, int, int]:
    """(num_chunks, floats of partial outputs, floats of partial max/sum)."""
    chunks = max(1, -(-max_seq_len // decode_chunk(head_dim)))
    return chunks, num_queries * num_heads * chunks * head_dim, num_queries * num_heads * chunks * 2


def decode_attention(q, q_stride, cache_layer, block_table, positions, token_row, num_heads, scale, window,
                     max_seq_len, workspace, out, kernel: str = "auto"):
    """Split-KV attention of ``positions.numel()`` single query tokens.  ``kernel``: "split" (one
    CTA per chunk of keys and kv head), "stream" (one persistent CTA per SM, TMA) or "auto" (stream
    when the step has enough keys to keep every SM's stream busy)."""
    from gllm_b200 import ops

    num_pages, _, hkv, block_size, d = cache_layer.shape
    n = positions.numel()
    parts = decode_stream_parts(d, num_heads, hkv, block_size, q, cache_layer) if kernel != "split" else 0
    if kernel == "stream" and not parts:
        raise ValueError(f"the stream decode kernel does not take {num_heads}/{hkv} heads of {d} with pages of "
                         f"{block_size}")
    spans = max(1, -(-max_seq_len // STREAM_SPAN))
    use_stream = bool(parts) and (kernel == "stream" or n * spans >= STREAM_MIN_ITEMS)
    if use_stream:
        chunks = spans
        n_o, n_ml = n * num_heads * spans * parts * d, n * num_heads * spans * parts * 2
        fn, name = _decode_stream_fn()[0], "attention_decode_stream"
    else:
        chunks, n_o, n_ml = decode_scratch_elems(n, num_heads, d, max_seq_len)
        fn, name = _decode_fn()[0], "attention_decode_bf16"
    if workspace is not None:
        part_o = workspace.get("attention_decode_partial_out", n_o, torch.float32)
        part_ml = workspace.get("attention_decode_partial_max_sum", n_ml, torch.float32)
    else:
        part_o = torch.empty(n_o, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(n_ml, dtype=torch.float32, device=q.device)
    code = fn(
        q.data_ptr(), q_stride, out.data_ptr(), out.stride(0), cache_layer.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), positions.data_ptr(), token_row.data_ptr(), n, part_o.data_ptr(),
        part_ml.data_ptr(), num_heads, hkv, d, block_size, num_pages, chunks, float(scale),
        int(window), ops.status_word(q.device).data_ptr(), ops._stream(),
    )
    ops._check(code, name)
    ops.launch_count += 1  # two kernels: split (or stream) and merge
    return out


def paged_attention_bf16(qkv, cache_layer, block_table, positions, token_row, num_heads, scale, window, batch, out):
    from gllm_b200 import ops

    n = qkv.shape[0]
    n_pf = batch.num_prefill_tokens
    d, block_size = cache_layer.shape[4], cache_layer.shape[3]
    if n_pf > 0 and batch.max_q_len >= TMEM_MIN_Q_LEN and prefill_tmem_supports(d, block_size, qkv, cache_layer):
        prefill_attention_tmem(qkv[:n_pf], qkv.shape[1], cache_layer, block_table, batch.cu_q, batch.context_lens,
                               batch.state_slots, batch.num_prefill_requests, batch.max_q_len, num_heads, scale,
                               window, out)
    elif n_pf > 0 and prefill_supports(d, block_size):
        prefill_attention(qkv, qkv.shape[1], cache_layer, block_table, batch.cu_q, batch.context_lens,
                          batch.state_slots, batch.num_prefill_requests, batch.max_q_len, num_heads, scale, window,
                          out)
    elif n_pf > 0:
        ops.paged_attention_simt(qkv[:n_pf], qkv.shape[1], cache_layer, block_table, positions[:n_pf],
                                 token_row[:n_pf], num_heads, scale, window, out[:n_pf])
    if n_pf < n:
        decode_attention(qkv[n_pf:], qkv.shape[1], cache_layer, block_table, positions[n_pf:], token_row[n_pf:],
                         num_heads, scale, window, batch.max_seq_len, batch.workspace, out[n_pf:])
    return out
