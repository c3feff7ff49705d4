"""Causal grouped-query attention over the paged cache.

The reference (gllm/model/layers/attention.py:122-182) runs three separate
projections, rotates q and k, scatters the new k, v into a flat cache, gathers
the whole padded context back out and calls a dense softmax(QK^T/sqrt(D)+bias)V.
Here: one product with the fused [q;k;v] weight, one kernel that rotates q and
k and stores k, v into their pages, one attention kernel that reads the pages
through the block table, one output product.  Query head ``h`` uses kv head
``h // (heads / kv_heads)`` (gllm/ops/attention/reference_attention.py:19-30).
"""

from __future__ import annotations

import math

import torch

from gllm_b200 import ops
from gllm_b200.parts.base import (
    POSITION_ENCODINGS,
    KVPageRequirement,
    Mixer,
    TensorExpectation,
    build_part,
    register_mixer,
)


@register_mixer("attention")
class Attention(Mixer):
    graph_safe_portions = True

    def __init__(self, names, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position=None, window: int | None = None, scale: float | None = None, bias: bool = False,
                 output_bias: bool = False, qk_norm_eps: float | None = None, qk_norm_unit_offset: bool = False):
        """``bias``: the q, k and v projections add a bias (tensor names ``q_bias``, ``k_bias``, ``v_bias``);
        ``output_bias``: so does the output projection (``o_bias``).  ``qk_norm_eps``: every head of q and of k
        is RMS-normed over its ``head_dim`` values before the rotation, with one weight each for all query heads
        and all key heads (``q_norm``, ``k_norm``).  Llama has none of the three (the reference's projections
        have no bias, gllm/model/layers/attention.py:139-142); they are here for architectures that do."""
        super().__init__(names)
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"head_dim {head_dim} is not supported: the attention kernels take multiples of 16 up to 256")
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.window = int(window) if window else None
        # the reference divides scores by head_dim ** 0.5 (reference_attention.py:40)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.position = build_part(POSITION_ENCODINGS, position) if position is not None else None
        self.bias, self.output_bias = bool(bias), bool(output_bias)
        self.qk_norm_eps = float(qk_norm_eps) if qk_norm_eps is not None else None
        self.qk_norm_unit_offset = bool(qk_norm_unit_offset)
        self.w_qkv: torch.Tensor | None = None
        self.w_o: torch.Tensor | None = None
        self.b_qkv: torch.Tensor | None = None
        self.b_o: torch.Tensor | None = None
        self.w_q_norm: torch.Tensor | None = None
        self.w_k_norm: torch.Tensor | None = None

    def kv_requirement(self):
        return KVPageRequirement.keys_and_values(self.num_kv_heads, self.head_dim, self.window)

    def kernel_needs(self):
        return {"attention_head_dims": {self.head_dim}}

    def expected_tensors(self):
        qd, kd = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        exp = {
            self.names["q"]: TensorExpectation((qd, self.hidden_size)),
            self.names["k"]: TensorExpectation((kd, self.hidden_size)),
            self.names["v"]: TensorExpectation((kd, self.hidden_size)),
            self.names["o"]: TensorExpectation((self.hidden_size, qd)),
        }
        if self.bias:
            exp[self.names["q_bias"]] = TensorExpectation((qd,), "bias")
            exp[self.names["k_bias"]] = TensorExpectation((kd,), "bias")
            exp[self.names["v_bias"]] = TensorExpectation((kd,), "bias")
        if self.output_bias:
            exp[self.names["o_bias"]] = TensorExpectation((self.hidden_size,), "bias")
        if self.qk_norm_eps is not None:
            exp[self.names["q_norm"]] = TensorExpectation((self.head_dim,), "vector")
            exp[self.names["k_norm"]] = TensorExpectation((self.head_dim,), "vector")
        if self.position is not None:
            exp.update(self.position.expected_tensors())
        return exp

    def load(self, get, dtype, device):
        q, k, v = (get(self.names[n], "matrix") for n in ("q", "k", "v"))
        self.w_qkv = torch.cat([q, k, v], dim=0).contiguous()
        self.w_o = get(self.names["o"], "matrix").contiguous()
        if self.bias:
            self.b_qkv = torch.cat([get(self.names[n], "bias") for n in ("q_bias", "k_bias", "v_bias")]).contiguous()
        if self.output_bias:
            self.b_o = get(self.names["o_bias"], "bias").contiguous()
        if self.qk_norm_eps is not None:
            self.w_q_norm = get(self.names["q_norm"], "vector").contiguous()
            self.w_k_norm = get(self.names["k_norm"], "vector").contiguous()
        if self.position is not None:
            self.position.load(get, dtype, device)

    def forward(self, x, ctx, cache):
        qkv = ops.linear(x, self.w_qkv, split_ok=True, bias=self.b_qkv)
        if self.qk_norm_eps is not None:
            qkv = ops.as_tensor(qkv)
            ops.rmsnorm_heads(qkv, self.w_q_norm, self.qk_norm_eps, 0, self.num_heads, self.head_dim,
                              self.qk_norm_unit_offset)
            ops.rmsnorm_heads(qkv, self.w_k_norm, self.qk_norm_eps, self.num_heads, self.num_kv_heads, self.head_dim,
                              self.qk_norm_unit_offset)
        view = ctx.groups[cache.group]
        rotary = self.position.rotary() if self.position is not None else None
        if self.position is not None and rotary is None:
            qkv = ops.as_tensor(qkv)
            self.position.apply(qkv, ctx, self.num_heads, self.num_kv_heads, self.head_dim)
        inv_freq, rotary_dim, interleaved = rotary if rotary is not None else (None, 0, False)
        pages = cache.kv_pages()
        qkv = ops.rope_store(
            qkv, ctx.positions, inv_freq,
            view.slot_mapping if cache.writes else None,
            pages, self.num_heads, self.num_kv_heads, self.head_dim, rotary_dim, interleaved,
        )
        attn = ops.paged_attention(
            qkv, pages, view.block_table, ctx.positions, ctx.token_row, self.num_heads, self.scale,
            window=self.window, batch=ctx,
        )
        return ops.linear(attn, self.w_o, split_ok=True, add_into=getattr(ctx, "residual_sink", None), bias=self.b_o)
