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


def test_every_declared_signature_belongs_to_its_library():
    """A function called through ctypes without its argument types gets its pointers cut
    to 32 bits: each table of signatures names functions of its own library only."""
    import re
    from pathlib import Path

    from fastgen_b200.csrc import build, ops

    csrc = Path(build.__file__).parent
    def exported(files):
        names = set()
        for f in files:
            names |= set(re.findall(r'extern "C" \w[\w\s\*]*?\b(fg_\w+)\(', (csrc / f).read_text()))
        return names
    core = exported(build.CORE_SOURCES)
    attn = exported(["attention.cu"])
    assert set(ops._CORE_SIGNATURES) <= core, set(ops._CORE_SIGNATURES) - core
    assert set(ops._ATTN_SIGNATURES) <= attn, set(ops._ATTN_SIGNATURES) - attn
    # and every exported function that takes a pointer is declared
    called = set(re.findall(r"\blib\.(fg_\w+)\(", Path(ops.__file__).read_text()))
    undeclared = called - set(ops._CORE_SIGNATURES) - set(ops._ATTN_SIGNATURES)
    int_only = {"fg_attention_decode_scratch_floats", "fg_attention_decode_split", "fg_attention_prefill_rows",
                "fg_attention_rows_per_block", "fg_last_error"}
    assert undeclared <= int_only, undeclared - int_only


def test_attention_tiles_are_in_ascending_order_of_keys():
    """The prompt kernels hand the tile list out from its end: the tiles that read the most
    keys come last in it, whatever the order of the sequences in the batch."""
    from fastgen_b200.engine.step import StepContext

    ctx = StepContext("cpu")
    # three sequences: 70 new tokens on 500 cached, one decoded token on 900, 130 new on none
    ctx.host_seq_slot = [4, 1, 7]
    ctx.host_seq_start = [0, 70, 71, 201]
    ctx.host_seq_cached = [500, 900, 0]
    tiles = ctx.attention_tiles(32, min_tokens=2)
    req, tok0, ntok = tiles.req.tolist(), tiles.tok0.tolist(), tiles.ntok.tolist()
    assert tiles.n == 3 + 5 and sorted(set(req)) == [4, 7]  # the single token is not a prompt tile
    start_of = {4: (0, 500), 7: (71, 0)}
    keys = [start_of[r][1] + (t - start_of[r][0]) + n for r, t, n in zip(req, tok0, ntok)]
    assert keys == sorted(keys)
    # every token of the two portions is in exactly one tile
    covered = sorted(t for t0, n in zip(tok0, ntok) for t in range(t0, t0 + n))
    assert covered == list(range(0, 70)) + list(range(71, 201))
    assert ctx.attention_tiles(32, min_tokens=2) is tiles  # cached per (tokens a tile, least tokens)
