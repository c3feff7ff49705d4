"""config.json files of the model sizes the benchmarks name (data, not code)."""

import json
import os

_DIR = os.path.dirname(os.path.abspath(__file__))


def preset_names() -> list[str]:
    return sorted(n[:-5] for n in os.listdir(_DIR) if n.endswith(".json"))


def load_preset(name: str) -> dict:
    path = os.path.join(_DIR, f"{name}.json")
    if not os.path.isfile(path):
        raise KeyError(f"no preset {name!r}; known: {preset_names()}")
    with open(path) as f:
        return json.load(f)
