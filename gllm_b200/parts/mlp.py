"""Dense gated feed-forward: ``down(silu(gate(x)) * up(x))``
(gllm/model/layers/mlp.py:44-47; the reference has no biases, ``bias=True`` adds one to each of the
three projections for checkpoints that have them).  The reference runs gate and up
as two products and the activation as separate elementwise calls; here their
weights are stacked and run as one product, in bfloat16 with the activation in
that product's epilogue (the weight is then stacked in alternating blocks of 64
gate and 64 up rows, which needs an intermediate size that is a multiple of 64)."""

from __future__ import annotations

import torch

from gllm_b200 import ops
from gllm_b200.parts.base import FeedForward, TensorExpectation, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    graph_safe_portions = True

    def __init__(self, names, hidden_size: int, intermediate_size: int, bias: bool = False):
        super().__init__(names)
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.bias = bool(bias)                            # tensor names gate_bias, up_bias, down_bias
        self.b_gate_up: torch.Tensor | None = None
        self.b_down: torch.Tensor | None = None
        self.w_gate_up: torch.Tensor | None = None
        self.w_down: torch.Tensor | None = None
        self.gated_blocks = False

    def expected_tensors(self):
        h, i = self.hidden_size, self.intermediate_size
        exp = {
            self.names["gate"]: TensorExpectation((i, h)),
            self.names["up"]: TensorExpectation((i, h)),
            self.names["down"]: TensorExpectation((h, i)),
        }
        if self.bias:
            exp[self.names["gate_bias"]] = TensorExpectation((i,), "bias")
            exp[self.names["up_bias"]] = TensorExpectation((i,), "bias")
            exp[self.names["down_bias"]] = TensorExpectation((h,), "bias")
        return exp

    def load(self, get, dtype, device):
        gate, up = get(self.names["gate"], "matrix"), get(self.names["up"], "matrix")
        # (with biases the activation cannot sit in the product's epilogue: the sums are not complete there)
        self.gated_blocks = (dtype == torch.bfloat16 and self.intermediate_size % ops.GATED_BLOCK == 0
                             and not self.bias)
        if self.gated_blocks:
            self.w_gate_up = ops.interleave_gate_up(gate, up)
        else:
            self.w_gate_up = torch.cat([gate, up], 0).contiguous()
        self.w_down = get(self.names["down"], "matrix").contiguous()
        if self.bias:
            self.b_gate_up = torch.cat([get(self.names["gate_bias"], "bias"), get(self.names["up_bias"], "bias")]).contiguous()
            self.b_down = get(self.names["down_bias"], "bias").contiguous()

    def forward(self, x, ctx):
        sink = getattr(ctx, "residual_sink", None)
        if self.gated_blocks:
            hidden = ops.linear_gated(x, self.w_gate_up)
        else:
            hidden = ops.silu_mul(ops.linear(x, self.w_gate_up, bias=self.b_gate_up))
        return ops.linear(hidden, self.w_down, split_ok=True, add_into=sink, bias=self.b_down)
