"""Reads a model folder's safetensors by tensor name and checks it against what
the model's parts expect.

The reference loads one ``model.safetensors`` and indexes the dict by
hard-wired names (gllm/model/model.py:79-86, gllm/model/layers/attention.py:55-61):
a missing tensor is a bare ``KeyError`` and shapes are not checked.  Here the
model first says which tensors it will read and their shapes; ``validate``
compares that with the file headers and raises ONE error that lists every
missing tensor, every unexpected tensor and every wrong shape.

dtype policy: matrices (operands of products, embedding tables) are held in the
run's dtype, bfloat16 or float32; vectors (norm weights) are held in fp32
whatever they were stored in; integer tables are int32.
"""

from __future__ import annotations

import json
import os
from typing import Mapping

import torch
from safetensors import safe_open

from gllm_b200.parts.base import TensorExpectation


class WeightError(ValueError):
    """The checkpoint does not hold what the model expects."""


class Checkpoint:
    """Lazy view of all ``*.safetensors`` files of a folder."""

    def __init__(self, folder: str):
        self.folder = os.fspath(folder)
        files = self._files()
        if not files:
            raise WeightError(f"no .safetensors file in {self.folder}")
        self._where: dict[str, str] = {}
        self._shapes: dict[str, tuple[int, ...]] = {}
        self._handles: dict[str, object] = {}
        for path in files:
            handle = safe_open(path, framework="pt", device="cpu")
            self._handles[path] = handle
            for name in handle.keys():
                if name in self._where:
                    raise WeightError(f"tensor {name!r} appears in two files of {self.folder}")
                self._where[name] = path
                self._shapes[name] = tuple(handle.get_slice(name).get_shape())

    def _files(self) -> list[str]:
        index = os.path.join(self.folder, "model.safetensors.index.json")
        if os.path.isfile(index):
            with open(index) as f:
                names = sorted(set(json.load(f)["weight_map"].values()))
            return [os.path.join(self.folder, n) for n in names]
        single = os.path.join(self.folder, "model.safetensors")
        if os.path.isfile(single):
            return [single]
        return sorted(
            os.path.join(self.folder, n) for n in os.listdir(self.folder) if n.endswith(".safetensors")
        )

    def names(self) -> list[str]:
        return sorted(self._where)

    def shape(self, name: str) -> tuple[int, ...]:
        return self._shapes[name]

    def tensor(self, name: str) -> torch.Tensor:
        return self._handles[self._where[name]].get_tensor(name)

    def validate(self, expected: Mapping[str, TensorExpectation], ignorable: tuple[str, ...] = ()) -> None:
        missing = sorted(n for n in expected if n not in self._where)
        unexpected = sorted(n for n in self._where if n not in expected and n not in ignorable)
        wrong = [
            (n, self._shapes[n], tuple(e.shape))
            for n, e in sorted(expected.items())
            if n in self._where and self._shapes[n] != tuple(e.shape)
        ]
        if not (missing or unexpected or wrong):
            return
        lines = [f"checkpoint {self.folder} does not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}):")
            lines += [f"    {n}  expected shape {list(expected[n].shape)}" for n in missing]
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}):")
            lines += [f"    {n}  shape {list(self._shapes[n])}" for n in unexpected]
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}):")
            lines += [f"    {n}  found {list(got)}, expected {list(want)}" for n, got, want in wrong]
        raise WeightError("\n".join(lines))

    def getter(self, dtype: torch.dtype, device: torch.device | str):
        """``get(name, role)`` for ``Part.load``: the tensor on ``device`` in the
        dtype its role asks for."""
        device = torch.device(device)

        def get(name: str, role: str = "matrix") -> torch.Tensor:
            t = self.tensor(name)
            if role in ("vector", "bias"):
                t = t.to(torch.float32)
            elif role == "int_table":
                t = t.to(torch.int32)
            elif role == "matrix":
                if not t.dtype.is_floating_point:
                    raise WeightError(f"tensor {name!r} is {t.dtype}, a floating-point matrix was expected")
                t = t.to(dtype)
            else:
                raise ValueError(f"unknown tensor role {role!r}")
            return t.to(device).contiguous()

        return get


def open_checkpoint(folder: str) -> Checkpoint:
    if not os.path.isdir(folder):
        raise WeightError(f"model folder {folder} does not exist")
    return Checkpoint(folder)
