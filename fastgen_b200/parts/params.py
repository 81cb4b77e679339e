"""Parameter dataclasses of the built-in parts.

Every size and constant a part needs is a field here; the parts read nothing
from the model they are in.  The architecture code fills these from the keys of
``config.json``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class Llama3Scaling:
    """Frequency rescaling of fastgen/forward.py:616-633."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_positions: int


@dataclass(frozen=True)
class RopeParams:
    """Rotary position encoding over adjacent pairs (fastgen/kernels/rope.py:77-89)."""

    head_dim: int
    theta: float
    scaling: Optional[Llama3Scaling] = None


@dataclass(frozen=True)
class NoPositionParams:
    """No position encoding: queries and keys are used as projected."""


@dataclass(frozen=True)
class AttentionParams:
    """Grouped-query causal attention (fastgen/model.py:50-80, forward.py:438-472).

    ``window`` is the number of most recent keys a query may see (itself
    included); ``None`` means all of them.  ``position`` is a ``PartSpec`` of a
    position encoding applied to queries and keys.  ``qk_layout`` says how the
    checkpoint orders the rows of a head in its query and key projections:
    ``"half_split"`` (the rotated pair of row ``j`` is row ``j + head_dim/2``, as
    Hugging Face Llama checkpoints store them; the rows are reordered at bind time,
    fastgen/utils/loading.py:296-305) or ``"adjacent"`` (pairs ``(2j, 2j+1)``, what the
    kernels rotate: taken as stored).
    """

    dim: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    position: object
    window: Optional[int] = None
    softmax_scale: Optional[float] = None  # None: head_dim ** -0.5 (forward.py:221)
    qk_layout: str = "adjacent"

    def __post_init__(self) -> None:
        if self.qk_layout not in ("adjacent", "half_split"):
            raise ValueError(f"qk_layout must be 'adjacent' or 'half_split', got {self.qk_layout!r}")
        if self.n_heads % self.n_kv_heads != 0:
            raise ValueError(
                f"{self.n_heads} query heads cannot be grouped over "
                f"{self.n_kv_heads} key/value heads"
            )
        if self.head_dim % 16 != 0 or not 16 <= self.head_dim <= 256:
            raise ValueError(
                f"head size {self.head_dim} is not supported: the attention "
                "kernels take multiples of 16 from 16 to 256"
            )
        if self.window is not None and self.window <= 0:
            raise ValueError(f"attention window must be positive, got {self.window}")


@dataclass(frozen=True)
class SwiGLUParams:
    """Dense gated feed-forward ``w2(silu(w1 x) * w3 x)`` (forward.py:491-496)."""

    dim: int
    ffn_dim: int


@dataclass(frozen=True)
class RMSNormParams:
    """``x * rsqrt(mean(x^2) + eps) * w`` (fastgen/kernels/rmsnorm.py:33-60)."""

    dim: int
    eps: float
