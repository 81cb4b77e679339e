"""Python face of the CUDA kernels: one :class:`Ops` per compute dtype.

Every method launches hand-written kernels on the current CUDA stream through
the C interface of the in-tree libraries.  The only library call is the bfloat16
matrix product (cuBLAS through ``torch.mm``), where the reference calls
``F.linear``; the float32 path uses this package's own float32 GEMM.  Nothing
here falls back to the CPU or to eager PyTorch.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_ulonglong, c_void_p
from typing import Optional

import torch

from . import build

FG_F32, FG_BF16 = 0, 1

STATUS_BAD_PAGE = 1
STATUS_BAD_TOKEN = 2
STATUS_WAIT_TIMEOUT = 4
STATUS_BAD_SPLITS = 8


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return FG_F32
    if dtype == torch.bfloat16:
        return FG_BF16
    raise TypeError(f"unsupported dtype {dtype}; the kernels take float32 and bfloat16")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_P, _I, _F = c_void_p, c_int, c_float

_CORE_SIGNATURES = {
    "fg_embedding": [_P, _I, _P, _P, _I, _I, _I, _I, _P, _P],
    "fg_rmsnorm": [_P, _I, _P, _I, _P, _I, _P, _I, _P, _I, _I, _F, _P],
    "fg_silu_gate": [_P, _P, _I, _I, _I, _I, _P],
    "fg_rope_kv_write": [_P, _I, _P, _I, _P, _I, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "fg_gemm_f32_nt": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _P],
    "fg_gemm_skinny_bf16": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _P],
    "fg_gemm_skinny_swiglu_bf16": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _P],
    "fg_gemm_skinny_qkv_bf16": [_P, _I, _P, _I, _P, _I, _I, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I,
                                _P, _P],
    "fg_sample": [_P, _I, _I, _I, _P, _F, c_ulonglong, _P, _P, _P, _P, _P, _P, _P],
    "fg_selftest_wait_timeout": [_I, _P, _P, _P],
    "fg_sample_uniform": [c_ulonglong, _P, _P, _P, _I, _P],
    "fg_make_kv_tensor_map": [_P, _P, _I, _I, _I, _I, _I, _I],
}

_ATTN_SIGNATURES = {
    "fg_attention_simt": [_P, _I, _P, _I, _I, _P, _P, _P, _I, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P, _P],
    "fg_attention_prefill_bf16": [_P, _I, _P, _I, _P, _P, _P, _I, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P, _P],
    "fg_attention_decode_bf16": [_P, _I, _P, _I, _P, _P, _P, _I, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P,
                                 ctypes.c_longlong, _I, _P, _P],
    "fg_attention_prefill_tma_bf16": [_P, _I, _P, _I, _P, _P, _I, _P, _I, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I,
                                      _I, _F, _P, _P],
    "fg_attention_prefill_tc5_bf16": [_P, _I, _P, _I, _P, _P, _I, _P, _I, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I,
                                      _I, _F, _P, _P, _P, _I, _I, _P, _I, _P, _P],
    "fg_attention_prefill_tc5_split_slots": [_I, _I, _I, _I, _I],
    "fg_attention_decode_tma_bf16": [_P, _I, _P, _I, _P, _P, _I, _P, _I, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I,
                                     _F, _P, ctypes.c_longlong, _I, ctypes.c_longlong, _P, _P],
    "fg_attention_decode_is_persistent": [_I, _I, _I, _I],
}

SKINNY_MAX_M = int(os.environ.get("FG_SKINNY_MAX_M", "8"))      # most tokens the weight-streaming product is used for (it takes up to 32)
SIMT_ROWS = 16       # query rows per block of the float32 attention kernel
PREFILL_ROWS = 64    # ... of the bfloat16 prompt kernel
PREFILL_TMA_ROWS = 128  # ... of the bfloat16 prompt kernel with tiled TMA loads
PREFILL_TMA_KEYS = 64   # key positions per tile of that kernel
DECODE_SPLIT = 128   # key positions per split of the bfloat16 single-token kernel


def _declare(lib: ctypes.CDLL, signatures) -> None:
    lib.fg_last_error.restype = ctypes.c_char_p
    for name, argtypes in signatures.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.argtypes = argtypes
        fn.restype = c_int


class KernelError(RuntimeError):
    pass


def describe_status(word: int) -> str:
    """The faults that the bits of a status word stand for, in words."""
    faults = []
    if word & STATUS_BAD_PAGE:
        faults.append("a block-table entry was missing or out of range")
    if word & STATUS_BAD_TOKEN:
        faults.append("a token id was outside the vocabulary")
    if word & STATUS_WAIT_TIMEOUT:
        faults.append("a bounded wait inside a kernel gave up")
    if word & STATUS_BAD_SPLITS:
        faults.append("decode attention was launched with too few splits")
    if word & ~(STATUS_BAD_PAGE | STATUS_BAD_TOKEN | STATUS_WAIT_TIMEOUT | STATUS_BAD_SPLITS):
        faults.append(f"unknown bits {word:#x}")
    return "kernel status: " + "; ".join(faults)


class TensorMap:
    """A 128-byte TMA descriptor kept on the host (64-byte aligned)."""

    def __init__(self) -> None:
        self._raw = ctypes.create_string_buffer(128 + 64)
        addr = ctypes.addressof(self._raw)
        self.ptr = (addr + 63) & ~63


def _check(lib: ctypes.CDLL, rc: int) -> None:
    if rc != 0:
        raise KernelError(lib.fg_last_error().decode())
    Ops.launches += 1


_core = None
_attn = {}


def core():
    global _core
    if _core is None:
        lib = build.core_library()
        _declare(lib, _CORE_SIGNATURES)
        _core = lib
    return _core


def attn(head_dim: int):
    lib = _attn.get(head_dim)
    if lib is None:
        lib = build.attention_library(head_dim)
        _declare(lib, _ATTN_SIGNATURES)
        lib.fg_attention_decode_scratch_floats.argtypes = [_I, _I, _I, ctypes.c_longlong]
        lib.fg_attention_decode_scratch_floats.restype = ctypes.c_longlong
        assert lib.fg_attention_rows_per_block() == SIMT_ROWS
        assert lib.fg_attention_prefill_rows() == PREFILL_ROWS
        assert lib.fg_attention_decode_split() == DECODE_SPLIT
        _attn[head_dim] = lib
    return lib


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError(
            f"fastgen_b200 runs on a CUDA device only (got {device}); there is no CPU path"
        )
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available; fastgen_b200 has no CPU path")
    return device


_device_index = 0  # set by Ops: the engine runs on one device
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  Asked for at every launch, so through torch's
    direct call where it has one (the public way costs several microseconds)."""
    if _raw_stream is not None:
        return _raw_stream(_device_index)
    return torch.cuda.current_stream().cuda_stream


def attention_tiling(n_heads: int, n_kv_heads: int, rows: int = SIMT_ROWS) -> int:
    """Tokens per attention tile for a head grouping and a block of ``rows``
    query rows (see attention.cu)."""
    group = n_heads // n_kv_heads
    return max(1, rows // min(group, rows))


class Ops:
    """Kernels bound to one compute dtype (``torch.float32`` or ``torch.bfloat16``).

    ``act_dtype`` is the type of activations, weights' matrices and the cache;
    the residual stream, norms' arithmetic, softmax and rotation angles are
    float32 in both modes.
    """

    launches = 0  # kernels of this package launched (graph replays add their kernels)

    def __init__(self, dtype: torch.dtype, device) -> None:
        self.device = require_cuda(device)
        global _device_index
        _device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.act_dtype = dtype
        self.code = _code(dtype)
        self.lib = core()
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._scratch = {}
        # the prompt attention kernel's blocks draw their work from it; zero between launches
        self._work_counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        # head size -> (partials, flags, (item, part) pairs they hold) of prompt-attention launches
        # that work on their long items in several parts; buffers that were outgrown stay alive, since
        # captured graphs may hold their addresses
        self._split = {}
        self._split_retired = []
        self.use_tcgen05 = not bool(os.environ.get("FG_NO_TCGEN05"))
        # library products accumulate and reduce in float32 (no bfloat16 split-K sums)
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

    # -- status word ---------------------------------------------------------
    def clear_status(self) -> None:
        """Zero the status word after a recorded fault, and with it what a kernel whose wait
        ran out may have left behind between launches: the prompt attention's work counter
        and the flags of its split items."""
        self.status.zero_()
        self._work_counter.zero_()
        for _scratch, flags, _room in self._split.values():
            flags.zero_()
        for _scratch, flags in self._split_retired:
            flags.zero_()

    def check_status(self) -> None:
        """Read the device status word (synchronises) and raise if a kernel
        recorded a fault instead of performing a bad access."""
        word = int(self.status.item())
        if word:
            self.status.zero_()
            raise KernelError(describe_status(word))

    def wait_timeout_selftest(self, limit: int = 1024):
        """Run a bounded wait on a barrier nobody arrives at (``limit`` polls) and return
        what the kernel saw: (first wait returned, second wait returned, cycles of the
        first, cycles of the second, wait on a completed phase returned).  The status word
        then holds the time-out bit."""
        out = torch.zeros(5, dtype=torch.int64, device=self.device)
        _check(self.lib, self.lib.fg_selftest_wait_timeout(int(limit), _ptr(self.status), _ptr(out), _stream()))
        return out.tolist()

    # -- kernels ---------------------------------------------------------------
    def embedding(self, table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        assert table.is_contiguous() and out.is_contiguous() and tokens.dtype == torch.int32
        n, dim = out.shape
        _check(self.lib, self.lib.fg_embedding(
            _ptr(table), _code(table.dtype), _ptr(tokens), _ptr(out), _code(out.dtype),
            n, dim, table.shape[0], _ptr(self.status), _stream()))
        return out

    def rmsnorm(self, h, weight, eps: float, out=None, delta=None, rows=None):
        """``h += delta`` (if given), then ``out = rmsnorm(h) * weight``.
        With ``out=None`` and a delta only the sum is done.  With ``rows``
        (int32 indices) only those rows are summed and normed into ``out``
        [len(rows), dim] and ``h`` is left as it was."""
        assert h.is_contiguous() and weight.is_contiguous()
        dim = h.shape[1]
        n = h.shape[0] if rows is None else rows.numel()
        if delta is not None:
            assert delta.is_contiguous() and delta.shape == h.shape
        if out is not None:
            assert out.is_contiguous() and out.shape == (n, dim)
        if rows is not None:
            assert rows.dtype == torch.int32 and out is not None
        _check(self.lib, self.lib.fg_rmsnorm(
            _ptr(h), _code(h.dtype), _ptr(delta), _code(delta.dtype) if delta is not None else 0,
            _ptr(weight), _code(weight.dtype), _ptr(out), _code(out.dtype) if out is not None else 0,
            _ptr(rows), n, dim, float(eps), _stream()))
        return out

    def linear(self, x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
               out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``x @ w.T`` for ``x`` [M, K] and ``w`` [N, K] (fastgen/forward.py:438-440)."""
        m, k = x.shape
        n = w.shape[0]
        assert w.shape[1] == k and x.stride(1) == 1 and w.stride(1) == 1
        if self.act_dtype == torch.float32:
            assert x.dtype == torch.float32 and w.dtype == torch.float32
            if out is None:
                out = torch.empty((m, n), dtype=torch.float32, device=x.device)
            assert out.dtype == torch.float32 and out.stride(1) == 1
            _check(self.lib, self.lib.fg_gemm_f32_nt(
                _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0),
                m, n, k, _stream()))
            return out
        assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
        want = out.dtype if out is not None else (out_dtype or torch.bfloat16)
        if (m <= SKINNY_MAX_M and k % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
            # few tokens: this package's weight-streaming kernel
            if out is None:
                out = torch.empty((m, n), dtype=want, device=x.device)
            assert out.stride(1) == 1
            _check(self.lib, self.lib.fg_gemm_skinny_bf16(
                _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), _code(out.dtype),
                m, n, k, _stream()))
            return out
        if want == torch.bfloat16:
            return torch.mm(x, w.t(), out=out) if out is not None else torch.mm(x, w.t())
        # float32 result of a bfloat16 product (logits)
        res = torch.mm(x, w.t(), out_dtype=torch.float32)
        if out is not None:
            out.copy_(res)
            return out
        return res

    def _skinny_ok(self, x: torch.Tensor, w: torch.Tensor, k: int) -> bool:
        return (x.dtype == torch.bfloat16 and x.shape[0] <= SKINNY_MAX_M and k % 8 == 0
                and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    def linear_swiglu(self, x: torch.Tensor, w13: torch.Tensor) -> Optional[torch.Tensor]:
        """``silu(x @ w1.T) * (x @ w3.T)`` in one kernel for a few tokens, for
        ``w13`` that holds w1 and w3 interleaved in blocks of 8 rows; ``None``
        when the shapes do not allow it (the caller then runs the product and
        the gate separately)."""
        m, k = x.shape
        f = w13.shape[0] // 2
        if f % 8 or not self._skinny_ok(x, w13, k):
            return None
        out = torch.empty((m, f), dtype=torch.bfloat16, device=x.device)
        _check(self.lib, self.lib.fg_gemm_skinny_swiglu_bf16(
            _ptr(x), x.stride(0), _ptr(w13), w13.stride(0), _ptr(out), out.stride(0), m, f, k, _stream()))
        return out

    def qkv_rope_write(self, x, wqkv, pos, req, freqs, memory, n_heads: int, n_kv_heads: int,
                       head_dim: int) -> Optional[torch.Tensor]:
        """Queries, keys and values of a few tokens in one kernel: the product
        against ``[wq; wk; wv]``, the rotation, and the write of keys and
        values into their pages.  Returns the rotated queries [T, heads*head_dim],
        or ``None`` when the shapes do not allow it."""
        m, k = x.shape
        if not self._skinny_ok(x, wqkv, k) or head_dim % 16:
            return None
        q = torch.empty((m, n_heads * head_dim), dtype=torch.bfloat16, device=x.device)
        _check(self.lib, self.lib.fg_gemm_skinny_qkv_bf16(
            _ptr(x), x.stride(0), _ptr(wqkv), wqkv.stride(0), _ptr(q), q.stride(0), m, k,
            _ptr(pos), _ptr(req), _ptr(freqs), _ptr(memory.k_pages), _ptr(memory.v_pages),
            _ptr(memory.block_table), memory.block_table.shape[1], memory.page_size,
            memory.k_pages.shape[0], n_heads, n_kv_heads, head_dim, _ptr(self.status), _stream()))
        return q

    def silu_gate(self, x13: torch.Tensor, out: torch.Tensor, interleave: int = 0) -> torch.Tensor:
        """``silu(gate) * up`` for ``x13`` holding gate and up as halves
        (``interleave=0``) or interleaved in blocks of 8 columns (``8``)."""
        n, two_f = x13.shape
        assert x13.is_contiguous() and out.is_contiguous() and out.shape == (n, two_f // 2)
        _check(self.lib, self.lib.fg_silu_gate(_ptr(x13), _ptr(out), _code(x13.dtype), n, two_f // 2,
                                               interleave, _stream()))
        return out

    def rope_kv_write(self, q, k, v, pos, req, freqs, k_pages, v_pages, block_table,
                      page_size: int, n_heads: int, n_kv_heads: int, head_dim: int) -> None:
        """Rotate ``q`` in place; rotate ``k`` and copy ``v`` into their pages.
        ``q``/``k``/``v`` are row-strided views [T, heads*head_dim]; ``k``/``v``
        may both be ``None`` (queries only)."""
        t = q.shape[0]
        assert q.stride(1) == 1 and pos.dtype == torch.int32 and req.dtype == torch.int32
        if k is not None:
            assert k.stride(1) == 1 and v.stride(1) == 1
            assert k_pages.is_contiguous() and v_pages.is_contiguous()
            assert block_table.dtype == torch.int32 and block_table.is_contiguous()
            n_pages = k_pages.shape[0]
            width = block_table.shape[1]
        else:
            n_pages = width = 0
        _check(self.lib, self.lib.fg_rope_kv_write(
            _ptr(q), q.stride(0), _ptr(k), k.stride(0) if k is not None else 0,
            _ptr(v), v.stride(0) if v is not None else 0, _code(q.dtype), _ptr(pos), _ptr(req),
            _ptr(freqs), _ptr(k_pages) if k is not None else None,
            _ptr(v_pages) if k is not None else None,
            _ptr(block_table) if k is not None else None, width, page_size, n_pages,
            t, n_heads, n_kv_heads, head_dim, _ptr(self.status), _stream()))

    def _decode_scratch(self, floats: int) -> torch.Tensor:
        """Scratch for the split partials.  Buffers are kept for good (captured
        graphs hold their addresses) and come in power-of-two sizes."""
        size = 1 << max(16, (floats - 1).bit_length())
        buf = self._scratch.get(size)
        if buf is None:
            buf = self._scratch[size] = torch.empty(size, dtype=torch.float32, device=self.device)
        return buf

    def make_kv_tensor_maps(self, k_pool, v_pool, page_size: int):
        """Tensor maps of a key and a value pool [layers, pages, kv heads, page,
        head size], or ``None`` where the tiled-load kernels do not apply."""
        n_layers, n_pages, n_kv_heads, page, head_dim = k_pool.shape
        if (k_pool.dtype != torch.bfloat16 or head_dim % 64 != 0 or page_size < 8
                or page_size & (page_size - 1)):
            return None
        # the box (rows a TMA instruction brings) is part of the map: one pair of maps
        # for the single-token kernel (128 positions a split), one for the prompt
        # kernel (64 positions a tile)
        maps = []
        for box_rows in (min(page_size, DECODE_SPLIT), min(page_size, PREFILL_TMA_KEYS)):
            for pool in (k_pool, v_pool):
                tm = TensorMap()
                _check(self.lib, self.lib.fg_make_kv_tensor_map(
                    tm.ptr, _ptr(pool), n_layers, n_pages, n_kv_heads, page_size, head_dim, box_rows))
                Ops.launches -= 1  # not a kernel
                maps.append(tm)
        return tuple(maps)

    def _split_buffers(self, head_dim: int, items: int):
        """Partials and flags for a prompt-attention launch that wants to work on its long
        items in parts, ``items`` (item, part) pairs in all (0: it does not).  They grow to the largest launch seen, outside
        graph captures only: a capture that finds them too small records a launch that does
        not split."""
        scratch, flags, room = self._split.get(head_dim, (None, None, 0))
        if items > room and not torch.cuda.is_current_stream_capturing():
            if room:
                self._split_retired.append((scratch, flags))
            room = max(items, 2 * room)
            scratch = torch.empty(room * PREFILL_TMA_ROWS * (head_dim + 2), dtype=torch.float32, device=self.device)
            flags = torch.zeros(2 * room, dtype=torch.int32, device=self.device)
            self._split[head_dim] = (scratch, flags, room)
        return scratch, flags, room

    def attention(self, q, out, memory, ctx, n_heads: int, n_kv_heads: int, head_dim: int,
                  window: Optional[int], scale: float) -> None:
        """Paged causal attention of the step's query tokens; ``memory`` is the
        run's :class:`~fastgen_b200.cache.LayerMemory`, ``ctx`` the step's
        context.  bfloat16 runs on the tensor cores: prompt portions in one
        kernel, single tokens in a split-and-combine pair (with tiled TMA loads
        where the shapes allow); float32 runs one CUDA-core kernel for all."""
        lib = attn(head_dim)
        k_pages, v_pages, block_table, page_size = (
            memory.k_pages, memory.v_pages, memory.block_table, memory.page_size)
        assert q.stride(1) == 1 and out.stride(1) == 1
        common = (_ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1], page_size,
                  k_pages.shape[0], _ptr(ctx.pos))
        if q.dtype == torch.float32:
            tiles = ctx.attention_tiles(attention_tiling(n_heads, n_kv_heads, SIMT_ROWS), 1)
            _check(lib, lib.fg_attention_simt(
                _ptr(q), q.stride(0), _ptr(out), out.stride(0), FG_F32, *common,
                _ptr(tiles.req), _ptr(tiles.tok0), _ptr(tiles.ntok), tiles.n,
                n_heads, n_kv_heads, head_dim, int(window or 0), float(scale),
                _ptr(self.status), _stream()))
            return
        use_tma = memory.tensor_maps is not None
        rows = PREFILL_TMA_ROWS if use_tma else PREFILL_ROWS
        tiling = attention_tiling(n_heads, n_kv_heads, rows)
        tiles = ctx.attention_tiles(tiling, 2)
        if tiles.n and use_tma:
            # head sizes 64 and 128: tcgen05.mma with S and O in tensor memory; other
            # multiples of 64: mma.sync on the same TMA tiles (FG_NO_TCGEN05=1 forces that)
            args = (_ptr(q), q.stride(0), _ptr(out), out.stride(0), memory.tensor_maps[2].ptr,
                    memory.tensor_maps[3].ptr, memory.layer_index, _ptr(block_table), block_table.shape[1],
                    page_size, k_pages.shape[0], _ptr(ctx.pos), _ptr(tiles.req), _ptr(tiles.tok0),
                    _ptr(tiles.ntok), tiles.n, n_heads, n_kv_heads, head_dim, int(window or 0), float(scale))
            if head_dim in (64, 128) and self.use_tcgen05:
                max_keys = -1 if tiles.max_keys is None else tiles.max_keys
                # a captured list has padding: what a step of prompt tokens only would hold
                nominal = 0 if tiles.count is None else max(1, -(-q.shape[0] // tiling))
                want = lib.fg_attention_prefill_tc5_split_slots(tiles.n, n_heads, n_kv_heads, max_keys, nominal)
                scratch, flags, room = self._split_buffers(head_dim, want)
                _check(lib, lib.fg_attention_prefill_tc5_bf16(
                    *args, _ptr(self._work_counter), _ptr(scratch), _ptr(flags), room, max_keys,
                    _ptr(tiles.count), nominal, _ptr(self.status), _stream()))
            else:
                _check(lib, lib.fg_attention_prefill_tma_bf16(*args, _ptr(self.status), _stream()))
        elif tiles.n:
            _check(lib, lib.fg_attention_prefill_bf16(
                _ptr(q), q.stride(0), _ptr(out), out.stride(0), *common,
                _ptr(tiles.req), _ptr(tiles.tok0), _ptr(tiles.ntok), tiles.n,
                n_heads, n_kv_heads, head_dim, int(window or 0), float(scale),
                _ptr(self.status), _stream()))
        singles = ctx.single_tokens()
        if singles.n:
            max_splits = max(1, -(-singles.max_len // DECODE_SPLIT))
            tma = use_tma and n_heads // n_kv_heads <= 16
            # the persistent kernel numbers its partials by the (request, split) pairs that
            # exist: the scratch follows the keys in the cache, not requests x longest request
            pairs = 0
            if tma and lib.fg_attention_decode_is_persistent(singles.n, n_heads, n_kv_heads, page_size):
                pairs = min(singles.n * max_splits, singles.stretches(DECODE_SPLIT))
            floats = lib.fg_attention_decode_scratch_floats(singles.n, max_splits, n_heads, pairs)
            scratch = self._decode_scratch(floats)
            head = (_ptr(singles.req), _ptr(singles.tok), singles.n, n_heads, n_kv_heads, head_dim,
                    int(window or 0), float(scale), _ptr(scratch), scratch.numel(), max_splits)
            if tma:
                _check(lib, lib.fg_attention_decode_tma_bf16(
                    _ptr(q), q.stride(0), _ptr(out), out.stride(0), memory.tensor_maps[0].ptr,
                    memory.tensor_maps[1].ptr, memory.layer_index, _ptr(block_table),
                    block_table.shape[1], page_size, k_pages.shape[0], _ptr(ctx.pos), *head, pairs,
                    _ptr(self.status), _stream()))
            else:
                _check(lib, lib.fg_attention_decode_bf16(
                    _ptr(q), q.stride(0), _ptr(out), out.stride(0), *common, *head, _ptr(self.status), _stream()))
            Ops.launches += 1  # the combine kernel

    def sample(self, logits, temps, top_p: float, seed: int, req_keys, positions,
               out_tokens, out_logprobs=None, scratch=None, with_status: bool = False) -> torch.Tensor:
        """One token per row of ``logits`` into ``out_tokens``.  ``with_status``: the
        device status word is copied to ``out_tokens[rows]`` (one more entry), so that the
        host's read of the tokens also tells it whether a kernel of the step recorded a fault."""
        rows, vocab = logits.shape
        assert logits.dtype == torch.float32 and logits.stride(1) == 1
        assert out_tokens.dtype == torch.int32 and out_tokens.numel() >= rows + int(with_status)
        if temps is not None:
            assert temps.dtype == torch.float32 and scratch is not None
            assert scratch.numel() >= rows * vocab and scratch.dtype == torch.float32
        if req_keys is not None:
            assert req_keys.dtype == torch.int64 and positions.dtype == torch.int32
        _check(self.lib, self.lib.fg_sample(
            _ptr(logits), logits.stride(0), rows, vocab, _ptr(temps), float(top_p),
            int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(req_keys), _ptr(positions), _ptr(out_tokens),
            _ptr(out_logprobs), _ptr(scratch), _ptr(self.status) if with_status else None, _stream()))
        return out_tokens

    def sample_uniform(self, seed: int, req_keys, positions) -> torch.Tensor:
        n = req_keys.numel()
        out = torch.empty(n, dtype=torch.float32, device=self.device)
        _check(self.lib, self.lib.fg_sample_uniform(
            int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(req_keys), _ptr(positions), _ptr(out), n, _stream()))
        return out
