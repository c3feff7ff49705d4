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
    in fp32 whatever the compute dtype is.  "int_table": integer table, int32.
    """

    shape: tuple[int, ...]
    role: str = "matrix"


# ------------------------------------------------- what mixers ask of the cache
@dataclass(frozen=True)
class KVPageRequirement:
    """Keys and values of every token (or of a trailing window of tokens)."""

    num_kv_heads: int
    head_dim: int
    # None: all tokens stay.  w: a token at position p needs positions > p - w.
    window: int | None = None


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


@dataclass
class MixerCache:
    """What one plan entry's mixer may touch of the cache."""

    group: int | None = None              # key into StepContext.groups
    pages: torch.Tensor | None = None     # [pages, 2, kv_heads, block_size, head_dim]
    writes: bool = True                   # False: attends over another entry's pages
    state: torch.Tensor | None = None     # [max_batch_size + 1, *StateRequirement.shape]; last row: padding rows


# ------------------------------------------------------------------ part bases
class Part:
    """Base of all parts: named tensors in, device tensors held."""

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
    own last branch output with the (updated in place) residual stream."""

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, feed_forward_norm: Norm):
        super().__init__()
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm

    def parts(self) -> list[Part]:
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

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
