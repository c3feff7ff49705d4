"""Typed configuration: what config.json says (ModelConfig) and what the
caller chooses for generation (GeneratorParams)."""

from gllm_b200.config.generator_params import GeneratorParams
from gllm_b200.config.llama_config import LlamaConfig, RopeScaling
from gllm_b200.config.model_config import ConfigError, ModelConfig, load_config
from gllm_b200.config.registry import (
    ARCHITECTURES,
    Architecture,
    architecture_for,
    register_architecture,
)

__all__ = [
    "GeneratorParams",
    "ConfigError",
    "LlamaConfig",
    "ModelConfig",
    "RopeScaling",
    "load_config",
    "ARCHITECTURES",
    "Architecture",
    "architecture_for",
    "register_architecture",
]
