"""From a model folder to a loaded model: config.json names the architecture,
the registry gives its configuration class and spec builder, the generic
decoder builds the parts, and the checkpoint is validated and read by name."""

from __future__ import annotations

import torch

from gllm_b200.config.model_config import ModelConfig, load_config
from gllm_b200.config.registry import architecture_for
from gllm_b200.models.decoder import DecoderModel
from gllm_b200.weights.loader import open_checkpoint

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def resolve_dtype(name: str | None, config: ModelConfig) -> torch.dtype:
    return TORCH_DTYPES[name or config.dtype]


def load_model(folder: str, dtype: str | None = None, device: str | torch.device = "cuda:0"):
    """Returns ``(config, model)`` with weights on ``device``."""
    config = load_config(folder)
    arch = architecture_for(config.architecture)
    spec = arch.build_spec(config)
    model = DecoderModel(spec, resolve_dtype(dtype, config), device)
    if torch.device(device).type == "cuda":
        # the kernels this model will ask for are compiled now, side by side, if they are not built yet
        from gllm_b200 import ops

        ops.prepare(model.dtype, model.kernel_needs().get("attention_head_dims", ()))
    model.load(open_checkpoint(folder))
    return config, model
