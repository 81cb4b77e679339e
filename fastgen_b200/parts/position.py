"""Position encodings: rotary (with llama3 frequency scaling) and none."""

from __future__ import annotations

import math
from typing import Optional

import torch

from .base import PositionEncoding, register_position
from .params import NoPositionParams, RopeParams


def rope_frequencies(params: RopeParams) -> torch.Tensor:
    """Float32 table of ``head_dim/2`` rotation frequencies.

    ``freq_j = theta ** -(2j / head_dim)``; with llama3 scaling a frequency whose
    wavelength ``2*pi/freq`` exceeds ``old_ctx/low`` is divided by ``factor``, one
    between ``old_ctx/high`` and ``old_ctx/low`` is blended
    ``(1-x)*freq/factor + x*freq`` with ``x = (old_ctx/wavelen - low)/(high - low)``,
    and shorter wavelengths are kept (fastgen/forward.py:609-635).  All
    arithmetic is float32 tensor arithmetic, as there.
    """
    hd = params.head_dim
    pows = torch.arange(0, hd, 2, dtype=torch.float32) / hd
    freqs = 1.0 / (params.theta ** pows)
    sc = params.scaling
    if sc is None:
        return freqs
    wavelen = (2 * math.pi) / freqs
    low_wavelen = sc.original_max_positions / sc.low_freq_factor
    high_wavelen = sc.original_max_positions / sc.high_freq_factor
    x = sc.original_max_positions / wavelen - sc.low_freq_factor
    x = x / (sc.high_freq_factor - sc.low_freq_factor)
    blended = (1 - x) * freqs / sc.factor + x * freqs
    out = torch.where(wavelen > low_wavelen, freqs / sc.factor, freqs)
    mid = (wavelen >= high_wavelen) & (wavelen <= low_wavelen)
    return torch.where(mid, blended, out)


class Rope(PositionEncoding):
    """Rotation of adjacent pairs ``(x[2j], x[2j+1])`` by ``pos * freq_j``
    (fastgen/kernels/rope.py:57-89).  The kernels are table-driven, so another
    frequency law is another ``table()``."""

    params: RopeParams

    def __init__(self, spec) -> None:
        super().__init__(spec)
        self._table: Optional[torch.Tensor] = None

    def table(self, device) -> Optional[torch.Tensor]:
        if self._table is None or self._table.device != torch.device(device):
            self._table = rope_frequencies(self.params).to(device).contiguous()
        return self._table


class NoPosition(PositionEncoding):
    params: NoPositionParams

    def table(self, device) -> Optional[torch.Tensor]:
        return None


register_position("rope", Rope)
register_position("none", NoPosition)
