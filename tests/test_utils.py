"""The hash of a token list is the reference's (fastgen/utils/misc.py:9-16)."""
import random
import struct

import pytest

from fastgen_b200.utils.misc import hashints, xxh32_words


def test_known_values():
    # XXH32 of the empty input with seed 0 (the algorithm's published test value)
    assert xxh32_words([]) == 0x02CC5D05
    # values taken from the reference's function on this machine
    assert hashints([]) == 90033154
    assert hashints([1, 2, 3]) == 143415071
    assert hashints(list(range(17))) == 1777473219


def test_against_the_xxhash_package():
    xxhash = pytest.importorskip("xxhash")
    np = pytest.importorskip("numpy")
    rng = random.Random(5)
    for n in list(range(0, 24)) + [257, 4096]:
        vals = [rng.randrange(0, 1 << 31) for _ in range(n)]
        digest = xxhash.xxh32_digest(np.array(vals, dtype=np.uint32).view(np.uint8))
        assert hashints(vals) == struct.unpack("<I", digest)[0] & 0x7FFFFFFF
