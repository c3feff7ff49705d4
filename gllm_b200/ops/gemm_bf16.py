"""bf16 matrix products ``x @ W.T`` with fp32 accumulation.

Two backends stand behind ``linear_bf16``: the engine's own tcgen05 kernels
(``csrc/gemm_bf16.cu``) and the library product (cuBLAS through
``torch.matmul``), which is what the reference itself uses for every
projection (gllm/model/layers/linear.py:20).  ``set_backend`` chooses.
"""

from __future__ import annotations

import torch

_BACKEND = "library"


def set_backend(name: str) -> None:
    global _BACKEND
    if name not in ("library", "tcgen05"):
        raise ValueError("backend must be 'library' or 'tcgen05'")
    _BACKEND = name


def get_backend() -> str:
    return _BACKEND


def linear_bf16(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    if out.dtype == torch.bfloat16:
        torch.matmul(x, weight.t(), out=out)
    else:
        # fp32 logits from bf16 operands: accumulate and write in fp32
        out.copy_(torch.mm(x, weight.t(), out_dtype=torch.float32))
    return out
