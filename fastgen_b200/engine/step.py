"""The step function: one batch of (request, its next tokens) through the model.

The reference has two entry points, ``prefill`` for prompt portions given as
``(n0, n1)`` pairs and a graph-captured ``decode`` (fastgen/forward.py:518-606);
a decoded token is just the pair ``(len-1, 1)``.  Here there is one ``step``: a
batch may hold portions of prompts beside single decoded tokens, cut anywhere.
It runs only the tokens it is given, reads everything earlier from the cache,
writes the new keys and values, and returns float32 logits at the wanted places
only.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import os

import numpy as np
import torch

from ..cache import CacheManager, OutOfPages, RequestCache
from .model import Model


def _decode_graphs():
    from .decode_graph import DecodeGraphs

    return DecodeGraphs


@dataclass
class StepEntry:
    """A request's next tokens and the places among them whose logits are wanted."""

    request_id: object
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class AttentionTiles:
    """Device arrays that cut the step's tokens into attention tiles; ``max_keys`` is the
    most keys one of them reads where the host knows it (a captured graph serves every
    length and says ``None``).  A captured graph's lists have room for the most tiles a step
    of its shape can have, with the real ones at the end (padding entries have request -1);
    ``count`` is then a device int that says how many are real in this replay."""

    req: torch.Tensor
    tok0: torch.Tensor
    ntok: torch.Tensor
    n: int
    max_keys: Optional[int] = None
    count: Optional[torch.Tensor] = None


@dataclass
class SingleTokens:
    """The step's sequences of one token: their slots and token indices on the
    device, and on the host the longest of them (cached tokens + 1) and what is
    known of all their lengths: the lengths themselves, or (for a captured graph,
    which serves every length) ``keys_bound``, the most cached positions these
    sequences can hold together (0: unknown)."""

    req: Optional[torch.Tensor]
    tok: Optional[torch.Tensor]
    n: int
    max_len: int
    lengths: Optional[List[int]] = None
    keys_bound: int = 0
    _stretches: Dict[int, int] = field(default_factory=dict)

    def stretches(self, stretch: int) -> int:
        """An upper bound on the (sequence, stretch of ``stretch`` consecutive positions)
        pairs that hold keys of these sequences.  Kernels that cut a sequence's keys into
        fixed stretches and keep a partial result per pair size their scratch by it."""
        got = self._stretches.get(stretch)
        if got is None:
            per_seq = -(-self.max_len // stretch)
            got = self.n * per_seq
            if self.lengths is not None:
                got = sum(-(-n // stretch) for n in self.lengths)
            elif self.keys_bound:
                # a sequence that holds k positions (all of them, or a window's) reaches into
                # at most k / stretch + 2 stretches
                got = min(got, self.keys_bound // stretch + 2 * self.n)
            self._stretches[stretch] = got
        return got


class StepContext:
    """Everything about the step's batch that parts may need, on host and device.

    Per token (device int32 ``[T]``): ``tokens``, ``pos`` (position in its
    request), ``req`` (its request's slot: the row of the block tables and the
    index of the fixed-size state; negative = padding).
    Per sequence of the batch (host lists and device int32): ``seq_slot``,
    ``seq_start`` (first token index, ``[B+1]``), ``seq_cached`` (tokens already
    in the cache before this step).
    """

    def __init__(self, device) -> None:
        self.device = device
        self.n_tokens = 0
        self.n_seqs = 0
        self.n_want = 0
        self.tokens = self.pos = self.req = self.want_rows = None
        self.seq_slot = self.seq_start = self.seq_cached = None
        self.host_seq_slot: List[int] = []
        self.host_seq_start: List[int] = [0]
        self.host_seq_cached: List[int] = []
        self._tiles: Dict[Tuple[int, int], AttentionTiles] = {}
        self._singles: Optional[SingleTokens] = None

    def attention_tiles(self, tokens_per_tile: int, min_tokens: int = 1) -> AttentionTiles:
        """Tiles of at most ``tokens_per_tile`` consecutive tokens over the
        sequences that bring at least ``min_tokens`` tokens, in ascending order of
        the number of keys a tile reads."""
        key = (tokens_per_tile, min_tokens)
        tiles = self._tiles.get(key)
        if tiles is None:
            tiles = self._tiles[key] = self._build_tiles(tokens_per_tile, min_tokens)
        return tiles

    def host_tiles(self, tpt: int, min_tokens: int) -> List[Tuple[int, int, int, int]]:
        """The tiles as host tuples (keys the tile reads, slot, first token, tokens), ascending
        by the keys: the kernels hand out the list from its end, so the tiles with the most keys
        start first and the short ones fill the tail of the launch."""
        tiles = []
        for b, slot in enumerate(self.host_seq_slot):
            start, end = self.host_seq_start[b], self.host_seq_start[b + 1]
            if end - start < min_tokens:
                continue
            cached = self.host_seq_cached[b]
            for t in range(start, end, tpt):
                n_tok = min(tpt, end - t)
                tiles.append((cached + t - start + n_tok, slot, t, n_tok))
        tiles.sort(key=lambda tile: tile[0])
        return tiles

    def _build_tiles(self, tpt: int, min_tokens: int) -> AttentionTiles:
        tiles = self.host_tiles(tpt, min_tokens)
        req = [tile[1] for tile in tiles]
        tok0 = [tile[2] for tile in tiles]
        ntok = [tile[3] for tile in tiles]
        n = len(req)
        if n == 0:
            return AttentionTiles(None, None, None, 0)
        packed = torch.tensor(req + tok0 + ntok, dtype=torch.int32).to(self.device)
        return AttentionTiles(packed[:n], packed[n : 2 * n], packed[2 * n :], n, tiles[-1][0])

    def single_tokens(self) -> "SingleTokens":
        """The sequences that bring exactly one token (decoded tokens)."""
        if self._singles is None:
            req, tok, lengths = [], [], []
            for b, slot in enumerate(self.host_seq_slot):
                start, end = self.host_seq_start[b], self.host_seq_start[b + 1]
                if end - start == 1:
                    req.append(slot)
                    tok.append(start)
                    lengths.append(self.host_seq_cached[b] + 1)
            n = len(req)
            if n == 0:
                self._singles = SingleTokens(None, None, 0, 0)
            else:
                packed = torch.tensor(req + tok, dtype=torch.int32).to(self.device)
                self._singles = SingleTokens(packed[:n], packed[n:], n, max(lengths), lengths)
        return self._singles


class Engine:
    """A model, its cache and the step function over them."""

    def __init__(
        self,
        model: Model,
        page_size: int,
        n_pages: int,
        max_requests: int,
        max_length: Optional[int] = None,
        num_cuda_graphs: int = 16,
        use_graphs: Optional[bool] = None,
        max_step_tokens: Optional[int] = None,
    ) -> None:
        """``max_step_tokens``: steps of up to that many tokens that are not single tokens only
        (prompt portions, alone or beside decoded tokens) replay CUDA graphs too, captured per
        padded shape when first met (``engine/step_graph.py``); ``None``: such steps are launched
        kernel by kernel."""
        self.model = model
        self.ops = model.ops
        self.device = model.ops.device
        args = model.args
        if max_length is None:
            max_length = args.max_positions
        max_length = min(max_length, args.max_positions)
        self.max_length = max_length
        self.cache = CacheManager(
            model.cache_specs(),
            model.state_specs(),
            model.kv_from(),
            page_size=page_size,
            n_pages=n_pages,
            max_requests=max_requests,
            max_length=max_length,
            dtype=model.ops.act_dtype,
            device=self.device,
            tensor_map_factory=model.ops.make_kv_tensor_maps,
        )
        self.memories = [self.cache.memory(e) for e in range(len(args.schedule))]
        self.last_h2d_bytes = 0
        if use_graphs is None:
            use_graphs = not bool(os.environ.get("FG_NO_CUDA_GRAPHS"))
        use_graphs = use_graphs and all(b.mixer.graph_safe for b in model.blocks)
        # steps of single tokens replay a captured graph (as generate.py:296-347)
        self.graphs = _decode_graphs()(self, max_requests, num_cuda_graphs) if use_graphs else None
        self.step_graphs = None
        if self.graphs is not None and max_step_tokens:
            from .step_graph import StepGraphs

            self.step_graphs = StepGraphs(self, self.graphs, max_step_tokens)

    # -- requests --------------------------------------------------------------
    def admit(self, request_id) -> RequestCache:
        return self.cache.admit(request_id)

    def release(self, request_id) -> None:
        self.cache.release(request_id)

    def length(self, request_id) -> int:
        return self.cache.get(request_id).length

    # -- the step --------------------------------------------------------------
    def _validate(self, entries: Sequence[StepEntry]) -> List[RequestCache]:
        vocab = self.model.args.vocab_size
        seen = set()
        reqs = []
        for e in entries:
            if e.request_id in seen:
                raise ValueError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            req = self.cache.get(e.request_id)
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.request_id!r} brings no tokens")
            for tok in e.tokens:
                if not 0 <= int(tok) < vocab:
                    raise ValueError(
                        f"token id {tok} of request {e.request_id!r} is outside the vocabulary of {vocab}"
                    )
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise ValueError(
                        f"request {e.request_id!r} wants logits at place {w} of {n} tokens"
                    )
            if req.length + n > self.max_length:
                raise OutOfPages(
                    f"request {e.request_id!r} would reach {req.length + n} tokens, more than "
                    f"the {self.max_length} positions this engine was built for"
                )
            reqs.append(req)
        return reqs

    def host_context(self, entries: Sequence[StepEntry], reqs: Sequence[RequestCache]):
        """The step on the host: a context with the sequences' lists, and per token its id,
        position and slot, and the wanted rows."""
        ctx = StepContext(self.device)
        tokens, pos, rq, want = [], [], [], []
        for e, req in zip(entries, reqs):
            n = len(e.tokens)
            base = len(tokens)
            tokens.extend(int(t) for t in e.tokens)
            pos.extend(range(req.length, req.length + n))
            rq.extend([req.slot] * n)
            want.extend(base + int(w) for w in e.want)
            ctx.host_seq_slot.append(req.slot)
            ctx.host_seq_cached.append(req.length)
            ctx.host_seq_start.append(base + n)
        return ctx, tokens, pos, rq, want

    def build_context(self, entries: Sequence[StepEntry], reqs: Sequence[RequestCache], host=None) -> StepContext:
        ctx, tokens, pos, rq, want = host if host is not None else self.host_context(entries, reqs)
        t, b, nw = len(tokens), len(entries), len(want)
        packed = np.concatenate(
            [
                np.asarray(tokens, dtype=np.int32),
                np.asarray(pos, dtype=np.int32),
                np.asarray(rq, dtype=np.int32),
                np.asarray(want, dtype=np.int32),
                np.asarray(ctx.host_seq_slot, dtype=np.int32),
                np.asarray(ctx.host_seq_start, dtype=np.int32),
                np.asarray(ctx.host_seq_cached, dtype=np.int32),
            ]
        )
        dev = torch.from_numpy(packed).to(self.device)
        self.last_h2d_bytes = packed.nbytes
        o = 0
        ctx.tokens, o = dev[o : o + t], o + t
        ctx.pos, o = dev[o : o + t], o + t
        ctx.req, o = dev[o : o + t], o + t
        ctx.want_rows, o = dev[o : o + nw], o + nw
        ctx.seq_slot, o = dev[o : o + b], o + b
        ctx.seq_start, o = dev[o : o + b + 1], o + b + 1
        ctx.seq_cached, o = dev[o : o + b], o + b
        ctx.n_tokens, ctx.n_seqs, ctx.n_want = t, b, nw
        return ctx

    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run one batch.  Returns float32 logits ``[wanted, vocab]`` in the order
        of the entries and of their ``want`` lists, or ``None`` if nothing is
        wanted.  Raises :class:`OutOfPages` (before touching anything on the
        device) when the cache cannot take the new tokens."""
        if not entries:
            return None
        reqs = self._validate(entries)
        need = [0] * len(self.cache.groups)
        for e, req in zip(entries, reqs):
            for g, n in enumerate(self.cache.pages_needed(req, req.length + len(e.tokens))):
                need[g] += n
        free = self.cache.free_pages()
        if any(n > f for n, f in zip(need, free)):
            raise OutOfPages(f"the step needs {need} new pages per group, free: {free}")
        for e, req in zip(entries, reqs):
            self.cache.reserve(req, req.length + len(e.tokens))
        logits = self._run(entries, reqs)
        for e, req in zip(entries, reqs):
            self.cache.advance(req, req.length + len(e.tokens))
        return logits

    @torch.inference_mode()
    def step_reserved(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """The step for a caller that manages the cache itself (the scheduler):
        pages for the new tokens are already reserved and the caller records the
        new lengths afterwards."""
        if not entries:
            return None
        return self._run(entries, self._validate(entries))

    def _run(self, entries, reqs) -> Optional[torch.Tensor]:
        self.cache.flush_tables()
        if self.graphs is not None and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
            logits = self.graphs.run(
                [int(e.tokens[0]) for e in entries], [r.length for r in reqs], [r.slot for r in reqs]
            )
            self.last_h2d_bytes = self.graphs.last_h2d_bytes
            return logits
        host = self.host_context(entries, reqs)
        if self.step_graphs is not None:
            ctx, tokens, pos, rq, want = host
            n_singles = sum(1 for e in entries if len(e.tokens) == 1)
            key = self.step_graphs.shape_for(len(tokens), len(want), n_singles, len(entries))
            # a padded shape that is not much larger than the step: the padding is computed too
            if key is not None and key[0] - len(tokens) <= max(64, len(tokens) // 8):
                logits = self.step_graphs.run(key, ctx, tokens, pos, rq, want)
                self.last_h2d_bytes = self.step_graphs.last_h2d_bytes
                return logits
        ctx = self.build_context(entries, reqs, host)
        return self.model.forward(ctx, self.memories)
