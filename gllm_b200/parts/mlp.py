"""Dense gated feed-forward: ``down(silu(gate(x)) * up(x))``
(gllm/model/layers/mlp.py:44-47), no biases.  The reference runs gate and up
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

    def __init__(self, names, hidden_size: int, intermediate_size: int):
        super().__init__(names)
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.w_gate_up: torch.Tensor | None = None
        self.w_down: torch.Tensor | None = None
        self.gated_blocks = False

    def expected_tensors(self):
        h, i = self.hidden_size, self.intermediate_size
        return {
            self.names["gate"]: TensorExpectation((i, h)),
            self.names["up"]: TensorExpectation((i, h)),
            self.names["down"]: TensorExpectation((h, i)),
        }

    def load(self, get, dtype, device):
        gate, up = get(self.names["gate"], "matrix"), get(self.names["up"], "matrix")
        self.gated_blocks = dtype == torch.bfloat16 and self.intermediate_size % ops.GATED_BLOCK == 0
        if self.gated_blocks:
            self.w_gate_up = ops.interleave_gate_up(gate, up)
        else:
            self.w_gate_up = torch.cat([gate, up], 0).contiguous()
        self.w_down = get(self.names["down"], "matrix").contiguous()

    def forward(self, x, ctx):
        sink = getattr(ctx, "residual_sink", None)
        if self.gated_blocks:
            hidden = ops.linear_gated(x, self.w_gate_up)
        else:
            hidden = ops.silu_mul(ops.linear(x, self.w_gate_up))
        return ops.linear(hidden, self.w_down, split_ok=True, add_into=sink)
