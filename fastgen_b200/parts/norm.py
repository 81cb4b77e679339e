"""RMSNorm, fused with the residual sum that precedes it."""

from __future__ import annotations

from typing import List

import torch

from .base import Norm, WeightSpec, register_norm
from .params import RMSNormParams


class RMSNorm(Norm):
    """``x * rsqrt(mean(x^2) + eps) * w`` in float32 (fastgen/kernels/rmsnorm.py:33-60).

    The weight keeps the dtype it was stored in (a 32-bit weight stays 32-bit);
    the float32 path upcasts it.
    """

    params: RMSNormParams

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.names["weight"], (self.params.dim,), ("ones",))]

    def bind(self, tensors, ops) -> None:
        self.ops = ops
        w = tensors["weight"]
        if ops.act_dtype == torch.float32:
            w = w.float()
        self.weight = w.contiguous()

    def forward(self, x, out_dtype=None, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, x.shape[1]), dtype=out_dtype or self.ops.act_dtype, device=x.device)
        return self.ops.rmsnorm(x, self.weight, self.params.eps, out=out, rows=rows)

    def add_forward(self, h, delta, rows=None):
        """``h += delta`` in float32 (stored back unless ``rows`` gathers), then the norm."""
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, h.shape[1]), dtype=self.ops.act_dtype, device=h.device)
        return self.ops.rmsnorm(h, self.weight, self.params.eps, out=out, delta=delta, rows=rows)


register_norm("rmsnorm", RMSNorm)
