"""The description of a model as data.

An architecture does not subclass a model: it writes down which parts each
layer is made of (``LayerSpec``), with their sizes and constants as parameters
(``PartSpec``), and the order in which the layers run (``PlanEntry``).  The
generic decoder builds and runs whatever the description says, so one model
can have different mixers and feed-forwards in different layers, run a layer
twice, or let one layer read another's cache.

The reference hard-wires one layer class repeated ``num_layers`` times
(gllm/model/model.py:96-102) and one order (gllm/model/model.py:202-222).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    """A registered part kind, its constructor parameters, and the checkpoint
    tensor name of each weight it holds (local key -> tensor name)."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    names: dict[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: how its parts are arranged (``block``, a registered block
    kind) and the parts, by the names that block kind declares
    (``Block.part_kinds``).  The built-in pre-norm block declares ``mixer_norm``,
    ``mixer``, ``feed_forward_norm`` and ``feed_forward``; a block with one
    shared norm, with norms after its branches or without a feed-forward
    declares other names and needs no change here."""

    block: str
    parts: dict[str, PartSpec] = field(default_factory=dict)

    def __getattr__(self, name: str) -> PartSpec:
        # spec.mixer, spec.feed_forward_norm ...: the part of that name
        parts = object.__getattribute__(self, "parts")
        if name in parts:
            return parts[name]
        raise AttributeError(name)


@dataclass(frozen=True)
class PlanEntry:
    """One step of the layer loop.

    ``layer`` indexes ``ModelSpec.layers`` and may repeat.  A mixer that keeps
    keys and values (or a state) gets a cache of its own for every entry,
    unless ``reads_cache_of`` names an earlier entry: then this entry's mixer
    writes nothing and attends over that entry's cache.
    """

    layer: int
    reads_cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    layers: tuple[LayerSpec, ...]
    plan: tuple[PlanEntry, ...]
    final_norm: PartSpec
    # Checkpoint names of the embedding table and of the output head; a tied
    # head has ``head_name`` None and multiplies by the embedding table.
    embedding_name: str
    head_name: str | None
    eos_token_ids: tuple[int, ...] = ()
    # Optional constants around the layer stack (none of them is Llama's): the looked-up embedding
    # rows are multiplied by ``embedding_scale``; the logits are multiplied by ``logit_scale`` and
    # then capped softly, ``cap * tanh(logits / cap)``.
    embedding_scale: float | None = None
    logit_scale: float | None = None
    logit_softcap: float | None = None
    # Tensor names that a checkpoint may hold and the model does not read
    # (for instance a stored head beside tied embeddings).
    ignorable_names: tuple[str, ...] = ()

    def validate(self) -> None:
        for i, entry in enumerate(self.plan):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"plan entry {i} names layer {entry.layer}, the model has {len(self.layers)}")
            if entry.reads_cache_of is not None:
                j = entry.reads_cache_of
                if not 0 <= j < i:
                    raise ValueError(f"plan entry {i} reads the cache of entry {j}, which does not run before it")
                if self.plan[j].reads_cache_of is not None:
                    raise ValueError(f"plan entry {i} reads the cache of entry {j}, which owns none")
