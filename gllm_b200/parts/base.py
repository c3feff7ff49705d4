"""Interfaces of the parts a layer is put together from, and their registries.

A part knows its own sizes and constants (constructor parameters) and the
checkpoint names of its tensors; it never sees a model configuration and does
not know which model it is in.  Five kinds exist:

* ``Mixer``            mixes information between the tokens of a request
                       (attention here); may keep keys and values in cache
                       pages and/or a state of fixed size per request;
* ``FeedForward``      works on each token alone (dense here; routed experts
                       would be another kind);
* ``Norm``             normalises the residual stream before a mixer or a
                       feed-forward, fused with the residual add;
* ``PositionEncoding`` tells a mixer how positions enter;
* ``Block``            the arrangement of the four above in one layer.

The reference has one fixed class for each (gllm/model/layers/attention.py,
mlp.py, norm.py, gllm/model/transformer.py) that pulls its tensors out of the
checkpoint dict by a hard-wired name and reads the global config.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping

import torch


# ------------------------------------------------------------ what parts load
@dataclass(frozen=True)
class TensorExpectation:
    """Shape and role of one checkpoint tensor.

    role "matrix": operand of a matrix product or an embedding table, held in
    the compute dtype.  "vector": small per-channel tensor (norm weight), held
    in fp32 whatever the compute dtype is.  "bias": the bias of a projection, held in fp32
    as well (random weights draw it around zero, a vector around one).  "int_table": integer table, int32.
    """

    shape: tuple[int, ...]
    role: str = "matrix"


# ------------------------------------------------- what mixers ask of the cache
@dataclass(frozen=True)
class KVPageRequirement:
    """What a mixer keeps in cache pages for every token (or for a trailing
    window of tokens): a tuple of tensors, each ``(heads, width)`` elements per
    token.  Attention keeps two of equal shape (keys and values,
    ``keys_and_values``); a mixer that caches one latent vector per token
    declares ``((1, width),)``; keys and values of different widths are two
    entries of different shape.  Inside a page the tensors lie one after the
    other, each as ``[heads, block_size, width]``."""

    tensors: tuple[tuple[int, int], ...]
    # None: all tokens stay.  w: a token at position p needs positions > p - w.
    window: int | None = None

    def __post_init__(self):
        if not self.tensors or any(len(t) != 2 or t[0] <= 0 or t[1] <= 0 for t in self.tensors):
            raise ValueError("a page requirement names at least one (heads, width) tensor of positive sizes")

    @classmethod
    def keys_and_values(cls, num_kv_heads: int, head_dim: int, window: int | None = None) -> "KVPageRequirement":
        shape = (int(num_kv_heads), int(head_dim))
        return cls((shape, shape), window)

    @property
    def elements_per_token(self) -> int:
        return sum(h * w for h, w in self.tensors)


@dataclass(frozen=True)
class StateRequirement:
    """A tensor of fixed shape per live request (recurrent state and the like),
    zeroed when a request starts at position 0."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


# ------------------------------------------------------- the batch, as parts see it
@dataclass
class GroupView:
    """One cache group's view of the running batch."""

    block_size: int
    # [max_batch_size, max_blocks_per_request] int32, row = state slot
    block_table: torch.Tensor
    # [n_tokens] int32: page * block_size + offset of each token, -1 = no store
    slot_mapping: torch.Tensor


@dataclass
class StepContext:
    """Device-side description of one step's flat batch.

    Tokens of all requests lie one after another (no padding rows).  Request
    ``r`` owns tokens ``cu_q[r] .. cu_q[r+1]-1`` at positions
    ``context_lens[r] ..``; ``state_slots[r]`` is its row in block tables and
    state tensors.
    """

    num_tokens: int
    num_requests: int
    dtype: torch.dtype
    positions: torch.Tensor       # [n] int32
    token_row: torch.Tensor       # [n] int32: state slot of the token's request
    cu_q: torch.Tensor            # [r+1] int32
    context_lens: torch.Tensor    # [r] int32: tokens cached before this step
    state_slots: torch.Tensor     # [r] int32
    groups: dict[int, GroupView] = field(default_factory=dict)
    # host copies for launch geometry
    q_lens_host: tuple[int, ...] = ()
    context_lens_host: tuple[int, ...] = ()
    max_q_len: int = 0
    max_seq_len: int = 0
    # the flat batch holds all multi-token portions first, then the single tokens
    num_prefill_tokens: int = 0
    num_prefill_requests: int = 0
    # device scratch the attention kernels share (owned by the step function)
    workspace: Any = None
    # [max_batch_size + 1] int32: the token last sampled for each state slot (a token id < 0 in the
    # batch stands for it)
    sampled: Any = None
    # Set by a block around a part's call: the fp32 residual stream the part's result will be added
    # to.  A part may hand it to its last product (``ops.linear(..., add_into=ctx.residual_sink)``)
    # and return what that returns (``ops.ADDED`` when the product added itself); parts that ignore
    # it return their result as before.
    residual_sink: Any = None


@dataclass
class MixerCache:
    """What one plan entry's mixer may touch of the cache."""

    group: int | None = None              # key into StepContext.groups
    pages: torch.Tensor | None = None     # [pages, block_size * elements_per_token]: this entry's pool layer
    writes: bool = True                   # False: attends over another entry's pages
    state: torch.Tensor | None = None     # [max_batch_size + 1, *StateRequirement.shape]; last row: padding rows
    requirement: KVPageRequirement | None = None
    block_size: int = 0

    def tensor(self, index: int) -> torch.Tensor:
        """The ``index``-th tensor the mixer declared, as a view ``[pages, heads, block_size, width]``
        of the pool (token ``t`` of a page is ``[:, :, t]``)."""
        before = sum(h * w for h, w in self.requirement.tensors[:index]) * self.block_size
        heads, width = self.requirement.tensors[index]
        return self.pages.as_strided(
            (self.pages.shape[0], heads, self.block_size, width),
            (self.pages.stride(0), self.block_size * width, width, 1),
            self.pages.storage_offset() + before,
        )

    def kv_pages(self) -> torch.Tensor:
        """``[pages, 2 (k|v), kv_heads, block_size, head_dim]`` for a mixer that declared
        ``KVPageRequirement.keys_and_values``."""
        t = self.requirement.tensors
        if len(t) != 2 or t[0] != t[1]:
            raise ValueError("this cache does not hold keys and values of equal shape")
        return self.pages.view(self.pages.shape[0], 2, t[0][0], self.block_size, t[0][1])


# ------------------------------------------------------------------ part bases
class Part:
    """Base of all parts: named tensors in, device tensors held."""

    def kernel_needs(self) -> dict:
        """What the part will ask of the kernel modules, so that they can be compiled side by side
        before the first step: ``{"attention_head_dims": {64}}`` for an attention mixer."""
        return {}

    # True when ``forward`` takes everything that varies between steps of equal shape from device
    # memory (positions, lengths, slots: the tensors of the StepContext), never from its host-side
    # copies, and never waits for the device: such a part's prompt portions may be captured in a CUDA
    # graph and replayed for other lengths and contexts.  Decode steps are captured either way.
    graph_safe_portions = False

    def __init__(self, names: Mapping[str, str] | None = None):
        self.names = dict(names or {})

    def expected_tensors(self) -> dict[str, TensorExpectation]:
        """Checkpoint name -> expectation, for everything ``load`` will read."""
        return {}

    def load(self, get: Callable[[str, str], torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        """Fetch tensors with ``get(checkpoint_name, role)``: the result is
        already on ``device`` in the dtype its role asks for."""


class Norm(Part):
    def forward(self, branch, resid: torch.Tensor, dtype: torch.dtype,
                rows: torch.Tensor | None = None) -> torch.Tensor:
        """``resid += branch`` in place (fp32), return norm(resid) in ``dtype``.
        With ``rows``: only those rows, ``resid`` untouched.  ``branch`` is a
        tensor, None, or a ``gllm_b200.ops.SplitSum`` (a mixer's or
        feed-forward's last product left unsummed); a norm that cannot take
        the latter calls ``ops.as_tensor`` on it."""
        raise NotImplementedError


class PositionEncoding(Part):
    """How positions enter a mixer.  Encodings of the rotary family expose
    ``rotary()`` and are applied inside the fused rotate-and-store kernel;
    any other encoding overrides ``apply``."""

    def rotary(self):
        """(inv_freq fp32 [rotary_dim/2], rotary_dim, interleaved) or None."""
        return None

    def apply(self, qkv: torch.Tensor, ctx: StepContext, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        """Transform q and k inside ``qkv`` in place (non-rotary encodings)."""


class Mixer(Part):
    def kv_requirement(self) -> KVPageRequirement | None:
        return None

    def state_requirement(self) -> StateRequirement | None:
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: MixerCache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """Arrangement of a layer's parts.  ``forward`` gets the previous layer's
    not yet added branch output and the fp32 residual stream, and returns its
    own last branch output with the (updated in place) residual stream.

    A block kind declares the parts it is made of in ``part_kinds``: part name
    -> "mixer" | "feed_forward" | "norm", in the order they are loaded.  The
    decoder builds exactly those from a ``LayerSpec`` and hands them to the
    constructor by name; each becomes an attribute.  A block holds at most one
    mixer that asks for a cache (the plan gives every entry one cache)."""

    part_kinds: dict[str, str] = {}

    def __init__(self, **parts: Part):
        super().__init__()
        missing = [n for n in self.part_kinds if n not in parts]
        extra = [n for n in parts if n not in self.part_kinds]
        if missing or extra:
            raise ValueError(f"block {type(self).__name__}: missing parts {missing}, unexpected parts {extra}")
        self._part_names = list(self.part_kinds)
        for name in self._part_names:
            setattr(self, name, parts[name])

    def parts(self) -> list[Part]:
        return [getattr(self, n) for n in self._part_names]

    def cache_mixer(self) -> "Mixer | None":
        """The mixer whose cache requirement the plan entry serves (None: the block keeps nothing)."""
        mixers = [p for p in self.parts() if isinstance(p, Mixer)]
        if len(mixers) > 1:
            raise ValueError("a block holds at most one mixer")
        return mixers[0] if mixers else None

    def forward(self, branch, resid, ctx: StepContext, cache: MixerCache):
        raise NotImplementedError


# ------------------------------------------------------------------ registries
MIXERS: dict[str, type] = {}
FEED_FORWARDS: dict[str, type] = {}
NORMS: dict[str, type] = {}
POSITION_ENCODINGS: dict[str, type] = {}
BLOCKS: dict[str, type] = {}


def _register(table: dict[str, type], kind: str):
    def deco(cls):
        table[kind] = cls
        cls.kind = kind
        return cls

    return deco


def register_mixer(kind: str):
    return _register(MIXERS, kind)


def register_feed_forward(kind: str):
    return _register(FEED_FORWARDS, kind)


def register_norm(kind: str):
    return _register(NORMS, kind)


def register_position_encoding(kind: str):
    return _register(POSITION_ENCODINGS, kind)


def register_block(kind: str):
    return _register(BLOCKS, kind)


def build_part(table: dict[str, type], spec) -> Part:
    """Instantiate the registered class of ``spec.kind`` with its parameters."""
    try:
        cls = table[spec.kind]
    except KeyError:
        raise KeyError(f"no part of kind {spec.kind!r} is registered; known: {sorted(table)}") from None
    return cls(names=spec.names, **spec.params)
