"""Typed model description.

A model is described as data: a list of layers, each naming the kind and the
parameters of its mixer, feed-forward and norms, plus a *schedule* that says in
which order layers run (a layer may appear twice, and an entry may read the
cache written by an earlier entry instead of writing its own).

The reference describes a model with one flat ``ModelArgs`` dataclass that is
uniform over layers (fastgen/model.py:12-40); here every layer carries its own
parameters so that layers may differ.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence, Tuple


class ConfigError(ValueError):
    """A ``config.json`` that cannot be turned into a model description."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: what kind it is, its constants and its tensors.

    ``kind`` selects the implementation in the part registry, ``params`` is
    that implementation's own parameter dataclass and ``names`` maps the
    part's local weight names (``"wq"``) to checkpoint tensor names
    (``"model.layers.3.self_attn.q_proj.weight"``).
    """

    kind: str
    params: Any
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement (``block``) and its parts.

    Every layer has one mixer (it is what owns the layer's cache or state), one
    feed-forward and their two norms.  An arrangement that needs more parts (norms
    after the mixer and the feed-forward, a second feed-forward, ...) names them in
    ``extra`` as ``(name, role, spec)`` with ``role`` one of ``"norm"``,
    ``"feed_forward"``, ``"mixer"``; the block receives them as keyword arguments
    under ``name`` and their tensors are loaded like everybody's.  (A mixer given
    there gets no cache or state of its own.)
    """

    block: str
    mixer: PartSpec
    mixer_norm: PartSpec
    ffn: PartSpec
    ffn_norm: PartSpec
    extra: Tuple[Tuple[str, str, PartSpec], ...] = ()


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.

    ``layer`` indexes ``ModelArgs.layers``.  ``kv_from`` names an earlier
    schedule entry whose cache this run reads without writing one of its own;
    ``None`` gives the run a cache of its own.
    """

    layer: int
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class ModelArgs:
    architecture: str
    dim: int
    vocab_size: int
    max_positions: int
    tie_embeddings: bool
    embedding_name: str
    output_name: Optional[str]
    layers: Sequence[LayerSpec]
    schedule: Sequence[ScheduleEntry]
    final_norm: PartSpec
    stop_tokens: Sequence[int] = ()

    def __post_init__(self) -> None:
        n = len(self.layers)
        for pos, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < n:
                raise ConfigError(
                    f"schedule entry {pos} names layer {entry.layer}, "
                    f"but the model has {n} layers"
                )
            if entry.kv_from is not None:
                if not 0 <= entry.kv_from < pos:
                    raise ConfigError(
                        f"schedule entry {pos} reads the cache of entry "
                        f"{entry.kv_from}, which does not run before it"
                    )
                if self.schedule[entry.kv_from].kv_from is not None:
                    raise ConfigError(
                        f"schedule entry {pos} reads the cache of entry "
                        f"{entry.kv_from}, which has no cache of its own"
                    )
        if not self.tie_embeddings and self.output_name is None:
            raise ConfigError("an untied model needs an output tensor name")


def require(config: Mapping[str, Any], keys: Sequence[str], what: str) -> None:
    """Raise one error naming every key of ``keys`` that ``config`` lacks."""
    missing = [k for k in keys if k not in config]
    if missing:
        raise ConfigError(f"{what} is missing required keys: {', '.join(missing)}")


def positive_int(config: Mapping[str, Any], key: str) -> int:
    value = config[key]
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config key {key!r} must be a positive integer, got {value!r}")
    return value
