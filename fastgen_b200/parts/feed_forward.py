"""Dense SwiGLU feed-forward."""

from __future__ import annotations

from typing import List

import torch

from .base import FeedForward, WeightSpec, register_feed_forward
from .params import SwiGLUParams


class SwiGLU(FeedForward):
    """``w2(silu(w1 x) * w3 x)`` (fastgen/forward.py:491-496).  Gate and up run
    as one product against ``[w1; w3]``; the activation is computed in float32
    and rounded once."""

    params: SwiGLUParams

    def weight_specs(self) -> List[WeightSpec]:
        p = self.params
        return [
            WeightSpec(self.names["w1"], (p.ffn_dim, p.dim)),
            WeightSpec(self.names["w3"], (p.ffn_dim, p.dim)),
            WeightSpec(self.names["w2"], (p.dim, p.ffn_dim)),
        ]

    def bind(self, tensors, ops) -> None:
        self.ops = ops
        dt = ops.act_dtype
        self.w13 = torch.cat([tensors["w1"], tensors["w3"]], dim=0).to(dt).contiguous()
        self.w2 = tensors["w2"].to(dt).contiguous()

    def forward(self, x, ctx):
        ops = self.ops
        x13 = ops.linear(x, self.w13)
        if x.dtype == torch.bfloat16:
            # a few tokens: the gate is computed inside the down projection
            y = ops.linear_silu_gate(x13, self.w2)
            if y is not None:
                return y
        g = torch.empty((x.shape[0], self.params.ffn_dim), dtype=x.dtype, device=x.device)
        ops.silu_gate(x13, g)
        return ops.linear(g, self.w2)


register_feed_forward("swiglu", SwiGLU)
