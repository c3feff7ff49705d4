"""Random-weights mode: writes a model folder (config.json, model.safetensors)
from a configuration and a seed, so the loader path is the tested path.

The reference has no such mode (it always downloads a checkpoint,
gllm/model/model.py:79-83).  Every tensor the architecture's spec expects is
drawn in a fixed order from one seeded generator in fp32 and then rounded to
the configuration's dtype: matrices ~ N(0, std), vectors (norm weights)
``1 + N(0, norm_jitter)``.
"""

from __future__ import annotations

import json
import os

import torch
from safetensors.torch import save_file

from gllm_b200.config.model_config import ModelConfig
from gllm_b200.config.registry import architecture_for

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def expected_tensors_of(config: ModelConfig):
    """Checkpoint name -> TensorExpectation for ``config``'s architecture,
    in the order the model's parts declare them."""
    from gllm_b200.models.decoder import expected_tensors_of_spec

    spec = architecture_for(config.architecture).build_spec(config)
    return expected_tensors_of_spec(spec)


def random_tensors(
    config: ModelConfig,
    seed: int,
    std: float = 0.02,
    norm_jitter: float = 0.0,
    std_overrides: dict[str, float] | None = None,
) -> dict[str, torch.Tensor]:
    gen = torch.Generator(device="cpu").manual_seed(int(seed))
    dtype = _TORCH_DTYPES[config.dtype]
    out: dict[str, torch.Tensor] = {}
    for name, exp in expected_tensors_of(config).items():
        if exp.role == "vector":
            t = torch.ones(exp.shape, dtype=torch.float32)
            if norm_jitter:
                t = t + torch.randn(exp.shape, generator=gen, dtype=torch.float32) * norm_jitter
        elif exp.role in ("matrix", "bias"):
            s = std
            for pattern, value in (std_overrides or {}).items():
                if pattern in name:
                    s = value
            t = torch.randn(exp.shape, generator=gen, dtype=torch.float32) * s
        else:
            raise ValueError(f"cannot draw a random tensor of role {exp.role!r} for {name}")
        out[name] = t.to(dtype).contiguous()
    return out


def write_random_model(
    folder: str,
    config: ModelConfig,
    seed: int,
    std: float = 0.02,
    norm_jitter: float = 0.0,
    std_overrides: dict[str, float] | None = None,
) -> str:
    """Write ``config.json`` and ``model.safetensors`` into ``folder``."""
    os.makedirs(folder, exist_ok=True)
    tensors = random_tensors(config, seed, std=std, norm_jitter=norm_jitter, std_overrides=std_overrides)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=1)
    save_file(tensors, os.path.join(folder, "model.safetensors"), metadata={"format": "pt", "seed": str(seed)})
    return folder
