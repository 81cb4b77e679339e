"""Arrangements of a layer's parts around the residual stream."""

from __future__ import annotations

from .base import Block, register_block


class PreNormBlock(Block):
    """``h = h + mixer(norm(h)); h = h + ffn(norm(h))`` (fastgen/forward.py:412-499).

    The residual stream is float32.  Each sum is fused into the norm that
    follows it, so the feed-forward's output is handed on as ``pending`` and
    added by the next layer's first norm (or by the model's final norm).
    """

    def forward(self, h, pending, ctx, memory):
        a = self.mixer_norm.add_forward(h, pending)
        m = self.mixer.forward(a, ctx, memory)
        f = self.ffn_norm.add_forward(h, m)
        return h, self.ffn.forward(f, ctx)


register_block("prenorm", PreNormBlock)
