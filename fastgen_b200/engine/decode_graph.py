"""CUDA graphs for steps in which every request brings exactly one token.

The reference captures ``decode`` once per batch-size bucket at start-up and
replays it with inputs copied into fixed tensors (fastgen/generate.py:300-347,
685-718; fastgen/forward.py:95-151).  The same here (``capture_all``; a bucket that was
not captured then is captured when a step first needs it): a bucket
of size ``n`` owns fixed device buffers for the tokens, positions and slots of
``n`` lanes; a step with fewer requests pads the rest with slot ``-1``, which
every kernel treats as "no request" (nothing is written to any page).
"""

from __future__ import annotations

import bisect
import gc
from typing import Dict, List, Optional, Sequence

import torch

from ..csrc.ops import Ops
from .step import AttentionTiles, SingleTokens, StepContext


def bucket_sizes(max_batch: int, num_graphs: int) -> List[int]:
    """``unique(round(linspace(1, max_batch, max(2, num_graphs))))`` (generate.py:301-316)."""
    n = max(2, num_graphs)
    if max_batch <= 1:
        return [1]
    sizes = {int(round(1 + i * (max_batch - 1) / (n - 1))) for i in range(n)}
    return sorted(sizes)


_RING = 8


class _Bucket:
    def __init__(self, size: int, max_len: int, keys_bound: int, device) -> None:
        self.size = size
        self.max_len = max_len  # positions the captured launch grids cover
        self.keys_bound = keys_bound  # cached positions the lanes can hold together
        # one packed buffer: tokens | pos | req | arange | ones
        # a ring of pinned staging buffers: a buffer is rewritten only after the
        # copy that last read it has run, so the host may run ahead of the device
        self.ring = [torch.empty(3 * size, dtype=torch.int32).pin_memory() for _ in range(_RING)]
        self.ring_events = [None] * _RING
        self.ring_next = 0
        self.dev = torch.zeros(5 * size, dtype=torch.int32, device=device)
        self.dev[2 * size : 3 * size] = -1  # until a step fills them, all lanes are padding
        self.dev[3 * size : 4 * size] = torch.arange(size, dtype=torch.int32, device=device)
        self.dev[4 * size :] = 1
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.n_kernels = 0

    def context(self, device) -> StepContext:
        n = self.size
        ctx = StepContext(device)
        ctx.tokens, ctx.pos, ctx.req = self.dev[:n], self.dev[n : 2 * n], self.dev[2 * n : 3 * n]
        ctx.want_rows = self.dev[3 * n : 4 * n]
        ctx.seq_slot = ctx.req
        ctx.n_tokens = ctx.n_seqs = ctx.n_want = n
        # every sequence is one token: one-token tiles for kernels that tile all
        # sequences, none for kernels that only take longer ones
        tiles = AttentionTiles(ctx.req, self.dev[3 * n : 4 * n], self.dev[4 * n :], n)
        none = AttentionTiles(None, None, None, 0)
        ctx.attention_tiles = lambda tokens_per_tile, min_tokens=1: tiles if min_tokens <= 1 else none
        singles = SingleTokens(ctx.req, self.dev[3 * n : 4 * n], n, self.max_len, None, self.keys_bound)
        ctx.single_tokens = lambda: singles
        return ctx


class DecodeGraphs:
    def __init__(self, engine, max_batch: int, num_graphs: int) -> None:
        # no reference back to the engine: graphs must not sit in a reference cycle,
        # or the garbage collector may destroy them while another capture is running
        self.model = engine.model
        self.memories = engine.memories
        self.device = engine.device
        self.sizes = bucket_sizes(max_batch, num_graphs)
        # A graph serves every context length: its launches cover the longest request the
        # cache admits, and kernels whose work follows the lengths (the persistent
        # single-token attention) read them from the positions.  The keys the cache can
        # hold bound the partial results of a step.
        self.max_len = engine.max_length
        self.cache_tokens = max((g.pool.n_pages * g.page_size for g in engine.cache.groups), default=0)
        self.buckets: Dict[int, _Bucket] = {}
        self.pool = None
        self.capture_stream = None
        self.warmed = set()  # batch sizes that ran once outside a capture
        self.replays = 0
        self.padded_replays = 0  # replays of a bucket larger than the step (lanes of slot -1)
        self.last_h2d_bytes = 0

    def run(self, tokens, positions: Sequence[int], slots: Sequence[int]) -> torch.Tensor:
        """Logits [n, vocab] of one decode step.  ``tokens`` is a list of ids, or
        a device int32 tensor (the previous step's samples, which then never
        visit the host)."""
        n = len(positions)
        size = self.sizes[bisect.bisect_left(self.sizes, n)]
        b = self._bucket(size)
        if b.graph is None:
            # before the step's inputs are copied in: the warm-up run and the capture see
            # padding lanes only (slot -1), so no request's keys, values or state are
            # touched by a forward pass that is not the step's own
            self._capture(b)
        slot = b.ring_next
        b.ring_next = (slot + 1) % _RING
        if b.ring_events[slot] is not None:
            b.ring_events[slot].synchronize()
        staging = b.ring[slot]
        host = staging.numpy()
        host[size : size + n] = positions
        host[size + n : 2 * size] = 0
        host[2 * size : 2 * size + n] = slots
        host[2 * size + n :] = -1
        if isinstance(tokens, torch.Tensor):
            b.dev[size : 3 * size].copy_(staging[size:], non_blocking=True)
            b.dev[:n].copy_(tokens[:n])
        else:
            host[:n] = tokens
            host[n:size] = 0
            b.dev[: 3 * size].copy_(staging, non_blocking=True)
        self.last_h2d_bytes = 4 * (2 * size if isinstance(tokens, torch.Tensor) else 3 * size)
        ev = torch.cuda.Event()
        ev.record()
        b.ring_events[slot] = ev
        b.graph.replay()
        Ops.launches += b.n_kernels
        self.replays += 1
        self.padded_replays += size > n
        return b.logits[:n]

    def _bucket(self, size: int) -> _Bucket:
        b = self.buckets.get(size)
        if b is None:
            b = self.buckets[size] = _Bucket(size, self.max_len, self.cache_tokens, self.device)
        return b

    def capture_all(self) -> None:
        """Capture the graph of every batch bucket now (the reference does so when it is
        built, fastgen/generate.py:300-347), so that no step waits for a capture."""
        for size in self.sizes:
            b = self._bucket(size)
            if b.graph is None:
                self._capture(b)

    def _capture(self, b: _Bucket) -> None:
        model, memories, size = self.model, self.memories, b.size
        b.dev[2 * size : 3 * size] = -1  # every lane is padding while warming up and capturing
        ctx = b.context(self.device)
        if size not in self.warmed:
            # once eagerly for a batch size (libraries load and choose their kernels,
            # function attributes get set), then capture
            model.forward(ctx, memories)
            self.warmed.add(size)
        b.graph, b.logits, b.n_kernels = self.capture(lambda: model.forward(ctx, memories))

    def capture(self, forward):
        """Capture ``forward()`` into a new graph of the shared memory pool.  Returns the graph,
        what ``forward`` returned and the number of this package's kernels in it."""
        graph = torch.cuda.CUDAGraph()
        before = Ops.launches
        # Captured by hand on a stream of its own: torch.cuda.graph() would also run the
        # collector and empty the allocator's cache, tens of milliseconds a capture, and
        # captures happen while requests are being served.  The collector stays off while
        # capturing: destroying an old graph or freeing device memory in the middle of a
        # capture would invalidate it.
        if self.capture_stream is None:
            self.capture_stream = torch.cuda.Stream(self.device)
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            self.capture_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.capture_stream):
                kw = {} if self.pool is None else {"pool": self.pool}
                graph.capture_begin(**kw)
                try:
                    result = forward()
                finally:
                    graph.capture_end()
            torch.cuda.current_stream().wait_stream(self.capture_stream)
        finally:
            if gc_was_on:
                gc.enable()
        if self.pool is None:
            self.pool = graph.pool()
        return graph, result, Ops.launches - before
