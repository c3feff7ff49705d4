"""Typed model configuration, read from the architecture's own config.json keys.

The reference builds its ``ModelConfig`` inline from ``config[key]`` lookups
(gllm/model/model.py:63-76, gllm/config/model_config.py:14-27): every key is
required, ``rope_scaling``, ``vocab_size``, ``tie_word_embeddings`` and
``architectures`` are never read.  Here every size and constant the model uses
comes from config.json through the ``from_dict`` of the configuration class that
the registry names for ``architectures[0]``; nothing is a literal in code.  This
module holds what every architecture shares; each architecture's own keys live
in a module of their own (``llama_config`` for ``LlamaForCausalLM``).
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any


class ConfigError(ValueError):
    """config.json is missing a key, or a value cannot be used."""


DTYPE_NAMES = {"bfloat16": "bfloat16", "float32": "float32"}


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's typed configuration."""

    architecture: str
    vocab_size: int
    hidden_size: int
    # "bfloat16" | "float32": the dtype the checkpoint names.
    dtype: str
    eos_token_ids: tuple[int, ...]

    def to_dict(self) -> dict[str, Any]:  # pragma: no cover - overridden
        raise NotImplementedError


def require(d: dict, key: str):
    if key not in d:
        raise ConfigError(f"config.json lacks required key {key!r}")
    return d[key]


def as_eos(value) -> tuple[int, ...]:
    # The reference accepts only a list (gllm/model/model.py:165-172: the int
    # branch repeats the list test); both forms are accepted here.
    if value is None:
        return ()
    if isinstance(value, bool):
        raise ConfigError("eos_token_id must be an int or a list of ints")
    if isinstance(value, int):
        return (value,)
    if isinstance(value, (list, tuple)) and all(isinstance(v, int) and not isinstance(v, bool) for v in value):
        return tuple(value)
    raise ConfigError("eos_token_id must be an int or a list of ints")


def load_config(source: str | os.PathLike | dict[str, Any]) -> ModelConfig:
    """Parse config.json (a folder, a file or an already-read dict) with the
    configuration class of the architecture it names."""
    from gllm_b200.config.registry import architecture_for

    if isinstance(source, dict):
        d = source
    else:
        path = os.fspath(source)
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        if not os.path.isfile(path):
            raise ConfigError(f"no config.json at {path}")
        with open(path, "r") as f:
            d = json.load(f)
    archs = d.get("architectures")
    if not archs or not isinstance(archs, list):
        raise ConfigError("config.json lacks 'architectures': cannot choose a model class")
    arch = architecture_for(archs[0])
    return arch.config_class.from_dict(d)
