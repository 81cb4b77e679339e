"""The sampler's entry point that allocates nothing, called through its exported
C symbol and compared with the ordinary entry point.

For callers that cannot get device memory when they sample (all memory already in
an arena of their own, a stream capture in progress, a loop that must not be stalled
by an allocation), ``fg_sample_noalloc`` works out of a fixed array inside the
library.  It must give exactly what ``fg_sample`` gives with a caller's buffer, also
when the array still holds what an earlier, different call left there.

This file sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _lib():
    from fastgen_b200.csrc import ops
    lib = ops.core()
    fn = lib.fg_sample_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_float,
                   ctypes.c_ulonglong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p]
    fn.restype = ctypes.c_int
    lib.fg_sample_noalloc_capacity.restype = ctypes.c_longlong
    return lib


def _both(lib, rows, vocab, seed, top_p, temp):
    from fastgen_b200.csrc.ops import Ops
    ops = Ops(torch.float32, DEV)
    g = torch.Generator().manual_seed(seed)
    logits = (torch.randn(rows, vocab, generator=g) * 2).to(DEV)
    temps = torch.full((rows,), temp, device=DEV)
    keys = torch.arange(rows, dtype=torch.int64, device=DEV) + seed
    posn = torch.arange(rows, dtype=torch.int32, device=DEV) * 3
    ref_tok = torch.empty(rows, dtype=torch.int32, device=DEV)
    ref_lp = torch.empty(rows, dtype=torch.float32, device=DEV)
    ops.sample(logits, temps, top_p, 99, keys, posn, ref_tok, ref_lp, torch.empty(rows * vocab, device=DEV))
    tok = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
    lp = torch.zeros(rows, dtype=torch.float32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.fg_sample_noalloc(logits.data_ptr(), logits.stride(0), rows, vocab, temps.data_ptr(), top_p, 99,
                               keys.data_ptr(), posn.data_ptr(), tok.data_ptr(), lp.data_ptr(), stream)
    assert rc == 0, lib.fg_last_error().decode()
    torch.cuda.synchronize()
    return tok, lp, ref_tok, ref_lp


def test_no_alloc_sampler_matches_the_ordinary_one_twice_in_a_row():
    lib = _lib()
    before = torch.cuda.memory_allocated()
    # two calls in a row with different shapes: the second finds the first one's leftovers
    for rows, vocab, seed, top_p, temp in ((7, 1000, 1, 0.9, 0.8), (3, 331, 2, 1.0, 1.3)):
        tok, lp, ref_tok, ref_lp = _both(lib, rows, vocab, seed, top_p, temp)
        assert torch.equal(tok, ref_tok)          # same kernel, same arithmetic: the same tokens
        assert torch.allclose(lp, ref_lp, rtol=0, atol=1e-6)
    del tok, lp, ref_tok, ref_lp
    assert torch.cuda.memory_allocated() <= before + (1 << 20)


def test_no_alloc_sampler_refuses_what_does_not_fit():
    lib = _lib()
    cap = lib.fg_sample_noalloc_capacity()
    assert cap == 1 << 20
    rows, vocab = 9, 128256  # 9 * 128256 > 2^20
    logits = torch.zeros(rows, vocab, device=DEV)
    tok = torch.empty(rows, dtype=torch.int32, device=DEV)
    rc = lib.fg_sample_noalloc(logits.data_ptr(), vocab, rows, vocab, None, 1.0, 0, None, None, tok.data_ptr(),
                               None, torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and "exceeds the built-in scratch" in lib.fg_last_error().decode()
    # what fits is served, greedy included
    rc = lib.fg_sample_noalloc(logits.data_ptr(), vocab, 8, vocab, None, 1.0, 0, None, None, tok.data_ptr(),
                               None, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(tok[:8].abs().sum()) == 0
