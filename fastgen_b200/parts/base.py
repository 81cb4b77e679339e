"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from a :class:`~fastgen_b200.config.PartSpec` alone: it knows
its own sizes, constants and tensor names and nothing about the model around it.
Parts are looked up by ``spec.kind`` in one registry per role, so a new mixer,
feed-forward, norm, position encoding or block arrangement is one ``register_*``
call and needs no change to the files of this package.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ..config.model_args import PartSpec


@dataclass(frozen=True)
class WeightSpec:
    """One checkpoint tensor a part needs.

    ``init`` is the law the random-weights writer draws it from:
    ``("normal", std)``, ``("ones",)``, ``("ones_jitter", half_width)`` for
    ``1 + U(-w, w)``, or ``("randint", high)`` for integer tables.
    ``integer`` tensors are kept as int32; others follow the compute dtype
    unless the file stores them in 32-bit (see ``weights.loader``).
    """

    name: str
    shape: Tuple[int, ...]
    init: tuple = ("normal", 0.02)
    integer: bool = False


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer that caches per-token entries needs per token.

    The usual case is keys and values: two pools of ``[pages, n_kv_heads, page, head_dim]``.
    ``n_pools = 1`` asks for one pool only (a mixer that keeps one entry per token, say a
    compressed one from which it makes keys and values itself); ``page_size`` asks for pages
    of that many tokens instead of the engine's.  Runs with equal specs share a group of
    pages; every group has its own pool of page ids and its own block table per request.
    """

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None  # keys a query may see, itself included
    n_pools: int = 2  # 2: keys and values; 1: one entry per token
    page_size: Optional[int] = None  # tokens per page; None: the engine's page size

    def __post_init__(self) -> None:
        if self.n_pools not in (1, 2):
            raise ValueError(f"a cache spec asks for 1 or 2 pools, got {self.n_pools}")
        if self.page_size is not None and self.page_size <= 0:
            raise ValueError(f"page size must be positive, got {self.page_size}")


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size per-request state of a mixer (float32, zeroed on admission)."""

    shape: Tuple[int, ...]


class Part:
    """Common base: weights are declared, then bound once they are on device."""

    def __init__(self, spec: PartSpec) -> None:
        self.spec = spec
        self.params = spec.params
        self.names = dict(spec.names)

    def weight_specs(self) -> List[WeightSpec]:
        return []

    def bind(self, tensors: Mapping[str, torch.Tensor], ops) -> None:
        """Receive the loaded tensors, keyed by local name, and the kernel set
        (``ops``) of the compute dtype.  Fused buffers are built here."""

    def tied_name(self, local: str) -> str:
        return self.names[local]


class Norm(Part):
    def forward(self, x: torch.Tensor, out_dtype=None, rows=None) -> torch.Tensor:
        """Normalise rows of ``x`` [T, dim] (only the rows indexed by the int32
        tensor ``rows`` when it is given)."""
        raise NotImplementedError

    def add_forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], rows=None) -> torch.Tensor:
        """``h += delta`` (32-bit sum; ``delta`` may be ``None``) and return
        ``norm(h)``.  With ``rows`` only those rows are computed and ``h`` may
        be left as it was.

        The default composes the two; implementations may fuse them."""
        if delta is not None:
            h.add_(delta.to(h.dtype))
        return self.forward(h, rows=rows)


class PositionEncoding(Part):
    """Position encoding of queries and keys.

    ``table()`` returns what the mixer's kernels need (for rotary encodings a
    float32 frequency table of ``head_dim/2`` entries, or ``None`` for no
    rotation)."""

    def table(self, device) -> Optional[torch.Tensor]:
        raise NotImplementedError


class Mixer(Part):
    #: whether ``forward`` only launches work that a CUDA graph may capture and
    #: copes with padding lanes (slot -1).  Steps of a model with a mixer that
    #: does not say so are never captured.
    graph_safe = False

    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, x: torch.Tensor, ctx, memory) -> torch.Tensor:
        """Mix tokens.  ``x`` is [T, dim] (normed), ``ctx`` the step's
        :class:`~fastgen_b200.engine.step.StepContext` and ``memory`` this
        run's :class:`~fastgen_b200.cache.LayerMemory`."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Block:
    """Arrangement of a layer's parts around the residual stream."""

    def __init__(self, mixer: Mixer, mixer_norm: Norm, ffn: FeedForward, ffn_norm: Norm, **extra: Part):
        self.mixer = mixer
        self.mixer_norm = mixer_norm
        self.ffn = ffn
        self.ffn_norm = ffn_norm
        #: further parts by name (``LayerSpec.extra``), for arrangements with more than four
        self.extra: Dict[str, Part] = dict(extra)

    def parts(self) -> Sequence[Part]:
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn, *self.extra.values())

    def forward(self, h, pending, ctx, memory):
        """Run the layer.  ``h`` is the residual stream [T, dim] (float32) and
        ``pending`` a delta not yet added to it (or ``None``); returns the new
        ``(h, pending)`` so that the sum can be fused with the next norm."""
        raise NotImplementedError


_MIXERS: Dict[str, Callable[[PartSpec], Mixer]] = {}
_FEED_FORWARDS: Dict[str, Callable[[PartSpec], FeedForward]] = {}
_NORMS: Dict[str, Callable[[PartSpec], Norm]] = {}
_POSITIONS: Dict[str, Callable[[PartSpec], PositionEncoding]] = {}
_BLOCKS: Dict[str, Callable[..., Block]] = {}


def register_mixer(kind: str, factory) -> None:
    _MIXERS[kind] = factory


def register_feed_forward(kind: str, factory) -> None:
    _FEED_FORWARDS[kind] = factory


def register_norm(kind: str, factory) -> None:
    _NORMS[kind] = factory


def register_position(kind: str, factory) -> None:
    _POSITIONS[kind] = factory


def register_block(kind: str, factory) -> None:
    _BLOCKS[kind] = factory


def _make(table, role: str, spec: PartSpec):
    factory = table.get(spec.kind)
    if factory is None:
        raise KeyError(
            f"no {role} of kind {spec.kind!r} is registered; known: {sorted(table)}"
        )
    return factory(spec)


def make_mixer(spec: PartSpec) -> Mixer:
    return _make(_MIXERS, "mixer", spec)


def make_feed_forward(spec: PartSpec) -> FeedForward:
    return _make(_FEED_FORWARDS, "feed-forward", spec)


def make_norm(spec: PartSpec) -> Norm:
    return _make(_NORMS, "norm", spec)


def make_position(spec: PartSpec) -> PositionEncoding:
    return _make(_POSITIONS, "position encoding", spec)


def make_block(kind: str, mixer, mixer_norm, ffn, ffn_norm, **extra) -> Block:
    factory = _BLOCKS.get(kind)
    if factory is None:
        raise KeyError(f"no block of kind {kind!r} is registered; known: {sorted(_BLOCKS)}")
    return factory(mixer, mixer_norm, ffn, ffn_norm, **extra)
