"""A small, whole LLM inference engine for one NVIDIA B200 (sm_100a).

The public surface mirrors TheEpicDolphin/gllm (gllm/engine/llm_engine.py,
gllm/engine/llm_engine_base.py, gllm/config/generator_params.py):
``LLMEngine``, ``GenerationRequest``, ``GenerationResult`` and
``GeneratorParams``.  Everything below them is built here: typed configuration,
architecture registry, safetensors loading, composable layer parts, a paged
cache manager, one step function, a scheduler, samplers and the CUDA kernels.
"""

__version__ = "0.1.0"

_LAZY = {
    "LLMEngine": ("gllm_b200.engine.llm_engine", "LLMEngine"),
    "GenerationRequest": ("gllm_b200.engine.request", "GenerationRequest"),
    "GenerationResult": ("gllm_b200.engine.request", "GenerationResult"),
    "GeneratorParams": ("gllm_b200.config.generator_params", "GeneratorParams"),
    "ModelConfig": ("gllm_b200.config.model_config", "ModelConfig"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib

        module, attr = _LAZY[name]
        return getattr(importlib.import_module(module), attr)
    raise AttributeError(f"module 'gllm_b200' has no attribute {name!r}")
