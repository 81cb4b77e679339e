"""Small helpers.

``hashints`` gives a list of token ids the 31-bit number the reference gives it
(fastgen/utils/misc.py:9-16: XXH32 with seed 0 over the ids as little-endian
32-bit words, the digest's four bytes read back in little-endian order, top bit
dropped), so that prompt hashes can be compared between the two engines' logs.
The hash is computed here in plain Python from the published XXH32 algorithm.
"""
from __future__ import annotations

from typing import Iterable

_P1, _P2, _P3, _P4, _P5 = 2654435761, 2246822519, 3266489917, 668265263, 374761393
_MASK = 0xFFFFFFFF


def _rotl(x: int, r: int) -> int:
    return ((x << r) | (x >> (32 - r))) & _MASK


def xxh32_words(words: Iterable[int], seed: int = 0) -> int:
    """XXH32 of a sequence of 32-bit words (their little-endian bytes)."""
    words = [w & _MASK for w in words]
    n = len(words)
    i = 0
    if n >= 4:
        v = [(seed + _P1 + _P2) & _MASK, (seed + _P2) & _MASK, seed & _MASK, (seed - _P1) & _MASK]
        while i + 4 <= n:
            for lane in range(4):
                v[lane] = (_rotl((v[lane] + words[i + lane] * _P2) & _MASK, 13) * _P1) & _MASK
            i += 4
        h = (_rotl(v[0], 1) + _rotl(v[1], 7) + _rotl(v[2], 12) + _rotl(v[3], 18)) & _MASK
    else:
        h = (seed + _P5) & _MASK
    h = (h + 4 * n) & _MASK
    for w in words[i:]:
        h = (_rotl((h + w * _P3) & _MASK, 17) * _P4) & _MASK
    h ^= h >> 15
    h = (h * _P2) & _MASK
    h ^= h >> 13
    h = (h * _P3) & _MASK
    h ^= h >> 16
    return h


def hashints(vals: Iterable[int]) -> int:
    """A non-negative hash below 2**31 of a list of ints (token ids)."""
    h = xxh32_words(vals)
    swapped = int.from_bytes(h.to_bytes(4, "big"), "little")
    return swapped & 0x7FFFFFFF
