"""CUDA graphs for steps that are not single tokens only: prompt portions, alone or beside
decoded tokens.

A step of a small model launches a hundred short kernels from Python, and the host needs longer
to launch them than the device to run them (measured: 2.8 ms of launching for a 1,024-token
step of a 16-layer model that computes for 2 ms).  The reference has the same cost and pays it
(its prefill is never captured, fastgen/generate.py:743-885).  Here such a step replays a graph
too.  A graph is captured for a *shape*: a number of tokens (the step is padded with tokens of
slot -1, which no kernel reads a page for or writes one for), a number of rows whose logits are
wanted, and a number of single-token sequences; everything else about a step is data: the
tokens, positions and slots, the tiles the attention kernels walk (lists padded with entries of
slot -1) and the single-token sequences.  All of it lives in one device buffer per shape and is
refreshed with one copy before the replay.

Shapes are rounded up to a few sizes, captured when a step first needs them; a step that fits
none (more tokens than the largest) runs eagerly.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..csrc.ops import Ops
from .step import AttentionTiles, SingleTokens, StepContext

_RING = 4
MAX_SHAPES = 24  # captured shapes kept; the least recently used one goes when another is needed


def token_buckets(max_tokens: int) -> List[int]:
    """Token counts a step is padded to: steps of 64 up to 512, of 256 up to 4,096, of 1,024 beyond."""
    sizes, t = [], 64
    while t < max_tokens:
        sizes.append(t)
        t += 64 if t < 512 else (256 if t < 4096 else 1024)
    sizes.append(max_tokens)
    return sizes


def _round_up(n: int, sizes: Sequence[int]) -> Optional[int]:
    for s in sizes:
        if n <= s:
            return s
    return None


class _Shape:
    """The fixed buffers and the graph of one step shape."""

    def __init__(self, n_tokens: int, n_want: int, n_singles: int, max_seqs: int, max_len: int, keys_bound: int,
                 device) -> None:
        self.n_tokens, self.n_want, self.n_singles = n_tokens, n_want, n_singles
        self.max_seqs, self.max_len, self.keys_bound = max_seqs, max_len, keys_bound
        self.device = device
        # tile lists are asked for by the kernels during the warm-up run: (tokens a tile, least
        # tokens of a sequence) -> offset of the list in the buffer
        self.tile_keys: Dict[Tuple[int, int], int] = {}
        self.tile_capacity: Dict[Tuple[int, int], int] = {}
        self.size = 0  # ints of the buffer in use
        self.off = {}
        for name, n in (("tokens", n_tokens), ("pos", n_tokens), ("req", n_tokens), ("want", n_want),
                        ("single_req", n_singles), ("single_tok", n_singles)):
            self.off[name] = self.size
            self.size += n
        self.capacity = self.size + 3 * 4 * (n_tokens + max_seqs + 8) + 4  # room for four tile lists
        self.dev = torch.zeros(self.capacity, dtype=torch.int32, device=device)
        self.ring = [torch.zeros(self.capacity, dtype=torch.int32).pin_memory() for _ in range(_RING)]
        self.ring_events: List[Optional[torch.cuda.Event]] = [None] * _RING
        self.ring_next = 0
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.n_kernels = 0

    def view(self, name: str, n: int) -> torch.Tensor:
        o = self.off[name]
        return self.dev[o : o + n]

    def tiles_for(self, tokens_per_tile: int, min_tokens: int) -> AttentionTiles:
        key = (tokens_per_tile, min_tokens)
        if key not in self.tile_keys:
            if self.graph is not None:
                raise RuntimeError(f"a captured step asked for a tile list {key} that its capture did not")
            # every sequence may end with a partial tile
            cap = -(-self.n_tokens // tokens_per_tile) + self.max_seqs
            if self.size + 3 * cap + 1 > self.capacity:
                raise RuntimeError("too many kinds of attention tiles in one step")
            self.tile_keys[key] = self.size
            self.tile_capacity[key] = cap
            self.dev[self.size : self.size + cap] = -1  # until a step fills them: no tile has a request
            self.size += 3 * cap + 1  # requests, first tokens, numbers of tokens, and how many tiles are real
        o, cap = self.tile_keys[key], self.tile_capacity[key]
        return AttentionTiles(self.dev[o : o + cap], self.dev[o + cap : o + 2 * cap], self.dev[o + 2 * cap : o + 3 * cap],
                              cap, None, self.dev[o + 3 * cap : o + 3 * cap + 1])

    def context(self) -> StepContext:
        ctx = StepContext(self.device)
        t = self.n_tokens
        ctx.tokens, ctx.pos, ctx.req = self.view("tokens", t), self.view("pos", t), self.view("req", t)
        ctx.want_rows = self.view("want", self.n_want)
        ctx.n_tokens, ctx.n_seqs, ctx.n_want = t, self.max_seqs, self.n_want
        ctx.attention_tiles = self.tiles_for
        if self.n_singles:
            singles = SingleTokens(self.view("single_req", self.n_singles), self.view("single_tok", self.n_singles),
                                   self.n_singles, self.max_len, None, self.keys_bound)
        else:
            singles = SingleTokens(None, None, 0, 0)
        ctx.single_tokens = lambda: singles
        return ctx


class StepGraphs:
    def __init__(self, engine, decode_graphs, max_tokens: int) -> None:
        # (no reference back to the engine: see DecodeGraphs)
        self.model = engine.model
        self.memories = engine.memories
        self.device = engine.device
        self.decode_graphs = decode_graphs  # shares its memory pool and capture stream
        self.max_seqs = engine.cache.max_requests
        self.max_len = engine.max_length
        self.keys_bound = decode_graphs.cache_tokens
        self.token_sizes = token_buckets(max_tokens)
        self.single_sizes = sorted({0, min(32, self.max_seqs), self.max_seqs})
        self.shapes: Dict[Tuple[int, int, int], _Shape] = {}
        self.replays = 0
        self.last_h2d_bytes = 0

    def shape_for(self, n_tokens: int, n_want: int, n_singles: int, n_seqs: int) -> Optional[Tuple[int, int, int]]:
        t = _round_up(n_tokens, self.token_sizes)
        if t is None or n_seqs > self.max_seqs:
            return None
        # wanted rows: as many as sequences (what generation asks for), or every token (replay)
        w = self.max_seqs if n_want <= self.max_seqs else t
        if n_want > w:
            return None
        return t, w, _round_up(n_singles, self.single_sizes)

    def run(self, key: Tuple[int, int, int], ctx_host: StepContext, tokens: Sequence[int], pos: Sequence[int],
            req: Sequence[int], want: Sequence[int]) -> Optional[torch.Tensor]:
        """Replay the graph of shape ``key`` for the step described by the host lists (and by
        ``ctx_host``'s sequences).  Returns logits ``[len(want), vocab]``."""
        sh = self.shapes.pop(key, None)
        if sh is None:
            while len(self.shapes) >= MAX_SHAPES:
                # every shape holds its graph's memory and a [rows, vocabulary] logits buffer
                old = self.shapes.pop(next(iter(self.shapes)))
                torch.cuda.current_stream().synchronize()  # its last replay is over
                old.graph = old.logits = None
            sh = _Shape(*key, self.max_seqs, self.max_len, self.keys_bound, self.device)
        self.shapes[key] = sh  # (most recently used last)
        if sh.graph is None:
            self._capture(sh)
        slot = sh.ring_next
        sh.ring_next = (slot + 1) % _RING
        if sh.ring_events[slot] is not None:
            sh.ring_events[slot].synchronize()
        staging = sh.ring[slot]
        host = staging.numpy()
        n, o = len(tokens), sh.off
        host[o["tokens"] : o["tokens"] + n] = tokens
        host[o["tokens"] + n : o["tokens"] + sh.n_tokens] = 0
        host[o["pos"] : o["pos"] + n] = pos
        host[o["pos"] + n : o["pos"] + sh.n_tokens] = 0
        host[o["req"] : o["req"] + n] = req
        host[o["req"] + n : o["req"] + sh.n_tokens] = -1  # padding tokens belong to no request
        host[o["want"] : o["want"] + len(want)] = want
        host[o["want"] + len(want) : o["want"] + sh.n_want] = 0
        if sh.n_singles:
            s_req, s_tok = [], []
            for b, slot_b in enumerate(ctx_host.host_seq_slot):
                if ctx_host.host_seq_start[b + 1] - ctx_host.host_seq_start[b] == 1:
                    s_req.append(slot_b)
                    s_tok.append(ctx_host.host_seq_start[b])
            k = len(s_req)
            host[o["single_req"] : o["single_req"] + k] = s_req
            host[o["single_req"] + k : o["single_req"] + sh.n_singles] = -1
            host[o["single_tok"] : o["single_tok"] + k] = s_tok
            host[o["single_tok"] + k : o["single_tok"] + sh.n_singles] = 0
        for (tpt, min_tokens), off in sh.tile_keys.items():
            cap = sh.tile_capacity[(tpt, min_tokens)]
            tiles = ctx_host.host_tiles(tpt, min_tokens)
            k = len(tiles)
            # the kernels hand the list out from its end: the padding goes to its front
            host[off : off + cap - k] = -1
            host[off + cap : off + 2 * cap - k] = 0
            host[off + 2 * cap : off + 3 * cap - k] = 0
            if k:
                host[off + cap - k : off + cap] = [tile[1] for tile in tiles]
                host[off + 2 * cap - k : off + 2 * cap] = [tile[2] for tile in tiles]
                host[off + 3 * cap - k : off + 3 * cap] = [tile[3] for tile in tiles]
            host[off + 3 * cap] = k
        sh.dev[: sh.size].copy_(staging[: sh.size], non_blocking=True)
        self.last_h2d_bytes = 4 * sh.size
        ev = torch.cuda.Event()
        ev.record()
        sh.ring_events[slot] = ev
        sh.graph.replay()
        Ops.launches += sh.n_kernels
        self.replays += 1
        return sh.logits[: len(want)] if want else None

    def _capture(self, sh: _Shape) -> None:
        model, memories = self.model, self.memories
        sh.dev[sh.off["req"] : sh.off["req"] + sh.n_tokens] = -1  # every token is padding while capturing
        if sh.n_singles:
            sh.dev[sh.off["single_req"] : sh.off["single_req"] + sh.n_singles] = -1
        ctx = sh.context()
        model.forward(ctx, memories)  # eagerly once: libraries choose their kernels, the tile lists get their places
        sh.graph, sh.logits, sh.n_kernels = self.decode_graphs.capture(lambda: model.forward(ctx, memories))
