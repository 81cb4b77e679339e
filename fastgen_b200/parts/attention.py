"""Grouped-query causal attention over the paged cache."""

from __future__ import annotations

from typing import List, Optional

import torch

from .base import CacheSpec, Mixer, WeightSpec, make_position, register_mixer
from .params import AttentionParams


def interleave_rope_rows(w: torch.Tensor, n_heads: int) -> torch.Tensor:
    """Reorder the rows of a q/k projection from the checkpoint's half-split
    rotary order to adjacent pairs: within a head, row ``2j`` <- row ``j`` and
    row ``2j+1`` <- row ``j + head_dim/2`` (the permutation the reference
    applies at load time, fastgen/utils/loading.py:296-305).  Scores are
    unchanged because queries and keys get the same permutation."""
    rows, cols = w.shape
    half = rows // n_heads // 2
    idx = torch.arange(rows, device=w.device).view(n_heads, 2, half)
    return w[idx.permute(0, 2, 1).reshape(-1)]


class GQAAttention(Mixer):
    """``wo(attention(rope(wq x), rope(wk x), wv x))`` (fastgen/forward.py:438-472).

    The three projections run as one product against ``[wq; wk; wv]`` built at
    bind time.  Keys and values of the step's tokens are written to this run's
    cache pages before attention reads them back, so a prompt portion attends to
    itself through the cache exactly as a decoded token does.
    """

    params: AttentionParams
    graph_safe = True

    def __init__(self, spec) -> None:
        super().__init__(spec)
        p = self.params
        self.position = make_position(p.position)
        self.scale = p.softmax_scale if p.softmax_scale is not None else p.head_dim ** -0.5
        self.q_width = p.n_heads * p.head_dim
        self.kv_width = p.n_kv_heads * p.head_dim

    def weight_specs(self) -> List[WeightSpec]:
        p = self.params
        return [
            WeightSpec(self.names["wq"], (self.q_width, p.dim)),
            WeightSpec(self.names["wk"], (self.kv_width, p.dim)),
            WeightSpec(self.names["wv"], (self.kv_width, p.dim)),
            WeightSpec(self.names["wo"], (p.dim, self.q_width)),
        ]

    def cache_spec(self) -> Optional[CacheSpec]:
        p = self.params
        return CacheSpec(p.n_kv_heads, p.head_dim, p.window)

    def bind(self, tensors, ops) -> None:
        p = self.params
        self.ops = ops
        dt = ops.act_dtype
        wq, wk = tensors["wq"], tensors["wk"]
        if p.qk_layout == "half_split":
            wq = interleave_rope_rows(wq, p.n_heads)
            wk = interleave_rope_rows(wk, p.n_kv_heads)
        self.wqkv = torch.cat([wq, wk, tensors["wv"]], dim=0).to(dt).contiguous()
        self.wo = tensors["wo"].to(dt).contiguous()
        self.freqs = self.position.table(ops.device)

    def forward(self, x, ctx, memory):
        p, ops = self.params, self.ops
        t = x.shape[0]
        q = None
        if memory.writes and x.dtype == torch.bfloat16:
            # a few tokens: projection, rotation and page write in one kernel
            q = ops.qkv_rope_write(x, self.wqkv, ctx.pos, ctx.req, self.freqs, memory,
                                   p.n_heads, p.n_kv_heads, p.head_dim)
        if q is None:
            if memory.writes:
                qkv = ops.linear(x, self.wqkv)
                q = qkv[:, : self.q_width]
                k = qkv[:, self.q_width : self.q_width + self.kv_width]
                v = qkv[:, self.q_width + self.kv_width :]
            else:
                # this run reads another run's cache: only queries are needed
                q = ops.linear(x, self.wqkv[: self.q_width])
                k = v = None
            ops.rope_kv_write(
                q, k, v, ctx.pos, ctx.req, self.freqs, memory.k_pages, memory.v_pages,
                memory.block_table, memory.page_size, p.n_heads, p.n_kv_heads, p.head_dim,
            )
        o = torch.empty((t, self.q_width), dtype=x.dtype, device=x.device)
        ops.attention(
            q, o, memory, ctx, p.n_heads, p.n_kv_heads, p.head_dim, p.window, self.scale,
        )
        return ops.linear(o, self.wo)


register_mixer("gqa_attention", GQAAttention)
