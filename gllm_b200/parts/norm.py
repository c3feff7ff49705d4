"""RMSNorm fused with the residual add.

``y = x / sqrt(mean(x^2) + eps) * w`` as gllm/model/layers/norm.py:20-22, with
eps inside the root and the weight multiplying directly.  The reference
computes the statistic in the input dtype; here it is fp32 always, over the
fp32 residual stream.  The add that the reference does separately before each
norm (gllm/model/transformer.py:58-59,72) happens in the same kernel.
"""

from __future__ import annotations

import torch

from gllm_b200 import ops
from gllm_b200.parts.base import Norm, TensorExpectation, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    graph_safe_portions = True

    def __init__(self, names, size: int, eps: float, unit_offset: bool = False):
        super().__init__(names)
        self.size = int(size)
        self.eps = float(eps)
        # True: the stored weight is an offset from one, y = x_hat * (1 + w)
        self.unit_offset = bool(unit_offset)
        self.weight: torch.Tensor | None = None

    def expected_tensors(self):
        return {self.names["weight"]: TensorExpectation((self.size,), "vector")}

    def load(self, get, dtype, device):
        self.weight = get(self.names["weight"], "vector")

    def forward(self, branch, resid, dtype, rows=None):
        return ops.add_rmsnorm(branch, resid, self.weight, self.eps, dtype, rows=rows, unit_offset=self.unit_offset)
