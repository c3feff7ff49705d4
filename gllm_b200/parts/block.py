"""Pre-norm arrangement: ``x += mixer(norm(x)); x += feed_forward(norm(x))``.

The reference defers each layer's last residual add to the next layer
(gllm/model/transformer.py:58-78): a layer receives the previous feed-forward
output and the residual, adds them, and returns its own feed-forward output
un-added.  The same protocol is kept here because it lets every add fuse into
the norm kernel that follows it.
"""

from __future__ import annotations

from gllm_b200 import ops
from gllm_b200.parts.base import Block, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    graph_safe_portions = True
    part_kinds = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def forward(self, branch, resid, ctx, cache):
        # a part may add its result into the residual itself (its last product's epilogue) and say so
        ctx.residual_sink = resid
        x = self.mixer_norm.forward(None if branch is ops.ADDED else branch, resid, ctx.dtype)
        mixed = self.mixer.forward(x, ctx, cache)
        x = self.feed_forward_norm.forward(None if mixed is ops.ADDED else mixed, resid, ctx.dtype)
        out = self.feed_forward.forward(x, ctx)
        ctx.residual_sink = None
        return out, resid
