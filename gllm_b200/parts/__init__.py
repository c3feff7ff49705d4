"""Layer parts: mixer, feed-forward, norm, position encoding and block."""

from gllm_b200.parts.base import (
    BLOCKS,
    FEED_FORWARDS,
    MIXERS,
    NORMS,
    POSITION_ENCODINGS,
    Block,
    FeedForward,
    GroupView,
    KVPageRequirement,
    Mixer,
    MixerCache,
    Norm,
    Part,
    PositionEncoding,
    StateRequirement,
    StepContext,
    TensorExpectation,
    build_part,
    register_block,
    register_feed_forward,
    register_mixer,
    register_norm,
    register_position_encoding,
)
from gllm_b200.parts import attention, block, mlp, norm, rotary  # noqa: F401  (register the built-in kinds)

__all__ = [
    "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS",
    "Block", "FeedForward", "GroupView", "KVPageRequirement", "Mixer", "MixerCache", "Norm", "Part",
    "PositionEncoding", "StateRequirement", "StepContext", "TensorExpectation", "build_part",
    "register_block", "register_feed_forward", "register_mixer", "register_norm", "register_position_encoding",
]
