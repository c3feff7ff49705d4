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

    @staticmethod
    def _normed(norm, part, branch, resid, ctx):
        """norm(resid + branch) for ``part``: lazily (for the part's first product to fuse) when the
        part takes that and nothing is left to add, else by the norm kernel."""
        if branch is ops.ADDED:
            branch = None
        x = norm.forward_lazy(branch, resid, ctx.dtype) if part.accepts_lazy_input else None
        return x if x is not None else norm.forward(branch, resid, ctx.dtype)

    def forward(self, branch, resid, ctx, cache):
        ctx.residual_sink = resid
        x = self._normed(self.mixer_norm, self.mixer, branch, resid, ctx)
        mixed = self.mixer.forward(x, ctx, cache)
        x = self._normed(self.feed_forward_norm, self.feed_forward, mixed, resid, ctx)
        out = self.feed_forward.forward(x, ctx)
        ctx.residual_sink = None
        return out, resid
