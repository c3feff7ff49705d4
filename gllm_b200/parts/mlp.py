"""Dense gated feed-forward: ``down(silu(gate(x)) * up(x))``
(gllm/model/layers/mlp.py:44-47), no biases.  The reference runs gate and up
as two products; here their weights are stacked and run as one."""

from __future__ import annotations

import torch

from gllm_b200 import ops
from gllm_b200.parts.base import FeedForward, TensorExpectation, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, names, hidden_size: int, intermediate_size: int):
        super().__init__(names)
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.w_gate_up: torch.Tensor | None = None
        self.w_down: torch.Tensor | None = None

    def expected_tensors(self):
        h, i = self.hidden_size, self.intermediate_size
        return {
            self.names["gate"]: TensorExpectation((i, h)),
            self.names["up"]: TensorExpectation((i, h)),
            self.names["down"]: TensorExpectation((h, i)),
        }

    def load(self, get, dtype, device):
        self.w_gate_up = torch.cat([get(self.names["gate"], "matrix"), get(self.names["up"], "matrix")], 0).contiguous()
        self.w_down = get(self.names["down"], "matrix").contiguous()

    def forward(self, x, ctx):
        gate_up = ops.linear(x, self.w_gate_up)
        return ops.linear(ops.silu_mul(gate_up), self.w_down, split_ok=True)
