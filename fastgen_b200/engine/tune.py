"""Memory budget -> cache size, after fastgen/utils/tune.py:31-84.

``cache_tokens = (gpu_gb*1e9 - weight bytes - prefill_gb*1e9) / bytes per cached
token``; ``prefill_tokens = prefill_gb*1e9 / (1.2 * per-token activation bytes)``
with the activation estimate of the reference: the residual stream twice plus
gate and up of the feed-forward (tune.py:45-55).
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class MemParams:
    cache_tokens: int
    prefill_tokens: int

    def round_to(self, n: int) -> None:
        self.cache_tokens = -(-self.cache_tokens // n) * n
        self.prefill_tokens = -(-self.prefill_tokens // n) * n


def mem_params(weight_bytes: int, bytes_per_cached_token: int, dim: int, widest_ffn: int,
               act_bytes: int, prefill_gb: float, gpu_gb: float) -> MemParams:
    prefill = int(prefill_gb * 1e9)
    avail = max(prefill, int(gpu_gb * 1e9) - weight_bytes)
    activation = int((2 * act_bytes * dim + 2 * act_bytes * widest_ffn) * 1.2)
    return MemParams(
        cache_tokens=(avail - prefill) // max(1, bytes_per_cached_token),
        prefill_tokens=prefill // max(1, activation),
    )
