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
        w1, w3 = tensors["w1"], tensors["w3"]
        f, d = w1.shape
        # gate and up rows interleaved in blocks of 8, so that 16 consecutive rows of
        # the fused weight are gate and up of the same 8 features (what the decode
        # kernel's epilogue needs); widths that are no multiple of 8 keep two halves
        self.interleave = 8 if f % 8 == 0 else 0
        if self.interleave:
            w13 = torch.stack([w1.view(f // 8, 8, d), w3.view(f // 8, 8, d)], dim=1).reshape(2 * f, d)
        else:
            w13 = torch.cat([w1, w3], dim=0)
        self.w13 = w13.to(dt).contiguous()
        self.w2 = tensors["w2"].to(dt).contiguous()

    def forward(self, x, ctx):
        ops = self.ops
        g = None
        if x.dtype == torch.bfloat16 and self.interleave:
            # a few tokens: product and gate in one kernel, the [gate | up] rows never exist
            g = ops.linear_swiglu(x, self.w13)
        if g is None:
            x13 = ops.linear(x, self.w13)
            g = torch.empty((x.shape[0], self.params.ffn_dim), dtype=x.dtype, device=x.device)
            ops.silu_gate(x13, g, self.interleave)
        return ops.linear(g, self.w2)


register_feed_forward("swiglu", SwiGLU)
