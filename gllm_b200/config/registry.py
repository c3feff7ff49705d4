"""One registry from an architecture's name to everything that builds it.

The reference's only "registry" is an enum of two hub ids
(gllm/model/model.py:22-24) and ``architectures`` in config.json is never
read.  Here ``config.json["architectures"][0]`` picks an ``Architecture``:
the class that parses that architecture's own config.json keys and the
function that turns the parsed configuration into a ``ModelSpec`` (the list of
layers, each put together from registered parts, and the order they run in).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable


@dataclass(frozen=True)
class Architecture:
    name: str
    # classmethod-like: dict (config.json) -> typed ModelConfig
    config_class: Any
    # ModelConfig -> gllm_b200.models.spec.ModelSpec
    build_spec: Callable[[Any], Any]


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class, build_spec) -> Architecture:
    """Add (or replace) an architecture.  Tests register toy ones this way."""
    arch = Architecture(name=name, config_class=config_class, build_spec=build_spec)
    ARCHITECTURES[name] = arch
    return arch


def _ensure_builtin_loaded() -> None:
    # The built-in architecture registers itself on import.
    import gllm_b200.models.llama  # noqa: F401


def architecture_for(name: str) -> Architecture:
    _ensure_builtin_loaded()
    try:
        return ARCHITECTURES[name]
    except KeyError:
        known = ", ".join(sorted(ARCHITECTURES)) or "(none)"
        raise KeyError(f"unknown architecture {name!r}; registered: {known}") from None
