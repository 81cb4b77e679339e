"""Each kernel alone against a plain float64 reference, at sizes other than the engine's."""

import math
import os
import random

import numpy as np
import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops32():
    from fastgen_b200.csrc.ops import Ops
    return Ops(torch.float32, DEV)


@pytest.fixture(scope="module")
def ops16():
    from fastgen_b200.csrc.ops import Ops
    return Ops(torch.bfloat16, DEV)


def _tol(dtype):
    return dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim,vocab", [(72, 331), (4096, 1000), (8, 5)])
def test_embedding(ops32, dtype, dim, vocab):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(vocab, dim, generator=g).to(DEV, dtype)
    tokens = torch.randint(0, vocab, (37,), generator=g).to(DEV, torch.int32)
    out = torch.empty(37, dim, dtype=torch.float32, device=DEV)
    ops32.embedding(table, tokens, out)
    assert torch.equal(out, table.float()[tokens.long()])
    bad = tokens.clone(); bad[3] = vocab
    ops32.embedding(table, bad, out)
    from fastgen_b200.csrc.ops import KernelError
    with pytest.raises(KernelError, match="vocabulary"):
        ops32.check_status()
    assert torch.count_nonzero(out[3]) == 0


@pytest.mark.parametrize("dim", [64, 200, 4096, 5000])
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
def test_rmsnorm(ops32, ops16, dim, wdtype):
    g = torch.Generator().manual_seed(dim)
    for ops, eps in ((ops32, 1e-5), (ops16, 1e-6)):
        act = ops.act_dtype
        h = (torch.randn(19, dim, generator=g) * 3).to(DEV)
        delta = torch.randn(19, dim, generator=g).to(DEV, act)
        w = (1 + 0.1 * torch.randn(dim, generator=g)).to(DEV, wdtype)
        ref_h = h.double() + delta.double()
        ref = pl.rmsnorm(ref_h, w.double(), eps)
        out = torch.empty(19, dim, dtype=act, device=DEV)
        h2 = h.clone()
        ops.rmsnorm(h2, w, eps, out=out, delta=delta)
        assert torch.allclose(h2.double(), ref_h, rtol=1e-6, atol=1e-6)  # the sum is float32
        assert torch.allclose(out.double(), ref, **_tol(act))
        # without delta; gathered rows leave h alone
        out1 = torch.empty(19, dim, dtype=act, device=DEV)
        ops.rmsnorm(h, w, eps, out=out1)
        assert torch.allclose(out1.double(), pl.rmsnorm(h.double(), w.double(), eps), **_tol(act))
        rows = torch.tensor([18, 0, 7, 7], dtype=torch.int32, device=DEV)
        outr = torch.empty(4, dim, dtype=act, device=DEV)
        h3 = h.clone()
        ops.rmsnorm(h3, w, eps, out=outr, delta=delta, rows=rows)
        assert torch.equal(h3, h)
        assert torch.allclose(outr.double(), ref[rows.long()], **_tol(act))


@pytest.mark.parametrize("m,n,k", [(1, 320, 192), (37, 200, 331), (130, 65, 17), (64, 64, 16), (3, 1000, 4096)])
def test_gemm_f32(ops32, m, n, k):
    g = torch.Generator().manual_seed(m * n)
    x = torch.randn(m, k, generator=g).to(DEV)
    w = torch.randn(n, k, generator=g).to(DEV)
    out = ops32.linear(x, w)
    ref = x.double() @ w.double().T
    assert torch.allclose(out.double(), ref, rtol=1e-5, atol=1e-4 * math.sqrt(k))
    # rows do not depend on what else is in the batch: bitwise
    out1 = ops32.linear(x[m // 2 : m // 2 + 1], w)
    assert torch.equal(out1[0], out[m // 2])
    # strided input (a column slice of a wider buffer)
    wide = torch.randn(m, k + 24, generator=g).to(DEV)
    assert torch.equal(ops32.linear(wide[:, 8 : 8 + k], w), ops32.linear(wide[:, 8 : 8 + k].contiguous(), w))


def test_linear_bf16(ops16):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(9, 200, generator=g).to(DEV, torch.bfloat16)
    w = torch.randn(331, 200, generator=g).to(DEV, torch.bfloat16)
    ref = x.double() @ w.double().T
    # float32 accumulation, one rounding to bfloat16 at the end (half an ulp = 2^-9 relative)
    err = (ops16.linear(x, w).double() - ref).abs()
    assert bool((err <= ref.abs() * 2.0 ** -8 + 1e-2).all()), float(err.max())
    out32 = ops16.linear(x, w, out_dtype=torch.float32)
    assert out32.dtype == torch.float32
    assert torch.allclose(out32.double(), ref, rtol=1e-4, atol=1e-3), float((out32.double() - ref).abs().max())


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("n,k", [(320, 192), (331, 200), (4096, 4096), (1000, 14336), (17, 72), (64, 8),
                                 (20011, 136), (16000, 520),   # these two: many more row blocks than the GPU holds blocks
                                 (6144, 4096), (5120, 3072), (5000, 72)])  # a little more than two blocks an SM: the shallow ring
def test_gemm_skinny(ops16, request, m, n, k):
    g = torch.Generator().manual_seed(m + n + k)
    x = torch.randn(m, k, generator=g).to(DEV, torch.bfloat16)
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).to(DEV, torch.bfloat16)
    ref = x.double() @ w.double().T
    from fastgen_b200.csrc import ops as O
    monkey = O.SKINNY_MAX_M
    O.SKINNY_MAX_M = 32  # the kernel takes up to 32 tokens; the engine uses it for fewer
    request.addfinalizer(lambda: setattr(O, "SKINNY_MAX_M", monkey))
    out32 = ops16.linear(x, w, out_dtype=torch.float32)
    assert out32.dtype == torch.float32
    assert torch.allclose(out32.double(), ref, rtol=1e-4, atol=2e-4), float((out32.double() - ref).abs().max())
    out16 = ops16.linear(x, w)
    err = (out16.double() - ref).abs()
    assert bool((err <= ref.abs() * 2.0 ** -8 + 1e-3).all()), float(err.max())
    # a row does not depend on the other rows of the batch: bitwise
    one = ops16.linear(x[m - 1 : m], w, out_dtype=torch.float32)
    assert torch.equal(one[0], out32[m - 1])
    # a column slice of a wider buffer as input, a wider buffer as output
    wide = torch.zeros(m, k + 16, dtype=torch.bfloat16, device=DEV)
    wide[:, 8 : 8 + k] = x
    assert torch.equal(ops16.linear(wide[:, 8 : 8 + k], w, out_dtype=torch.float32), out32)


@pytest.mark.parametrize("m", [1, 8, 11, 32])
@pytest.mark.parametrize("f,k", [(512, 192), (328, 200), (14336, 4096), (8, 72), (9000, 72)])
def test_gemm_skinny_swiglu(ops16, m, f, k):
    """Gate/up product with the gate in its epilogue, against product-then-gate."""
    g = torch.Generator().manual_seed(m * k + f)
    x = torch.randn(m, k, generator=g).to(DEV, torch.bfloat16)
    w1 = (torch.randn(f, k, generator=g) * 2 / math.sqrt(k)).to(torch.bfloat16)
    w3 = (torch.randn(f, k, generator=g) * 2 / math.sqrt(k)).to(torch.bfloat16)
    w13 = torch.stack([w1.view(f // 8, 8, k), w3.view(f // 8, 8, k)], dim=1).reshape(2 * f, k).to(DEV)
    from fastgen_b200.csrc import ops as O
    old, O.SKINNY_MAX_M = O.SKINNY_MAX_M, 32
    try:
        out = ops16.linear_swiglu(x, w13)
    finally:
        O.SKINNY_MAX_M = old
    assert out is not None and out.shape == (m, f)
    x1 = (x.double().cpu() @ w1.double().T).to(torch.bfloat16).double()   # each product rounded once
    x3 = (x.double().cpu() @ w3.double().T).to(torch.bfloat16).double()
    ref = x1 * torch.sigmoid(x1) * x3
    err = (out.double().cpu() - ref).abs()
    # one bfloat16 ulp of either product moves the result by about 2^-7 of it
    assert bool((err <= ref.abs() * 2.0 ** -6 + 2e-2).all()), float(err.max())
    # the separate gate kernel reads the same interleaved layout
    x13 = ops16.linear(x, w13)
    out2 = torch.empty(m, f, dtype=torch.bfloat16, device=DEV)
    ops16.silu_gate(x13, out2, 8)
    assert torch.allclose(out2.float(), out.float(), rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("m", [1, 5, 8, 20])
@pytest.mark.parametrize("hq,hkv,hd,page,dim", [(4, 1, 16, 8, 64), (6, 3, 32, 16, 192), (6, 2, 48, 8, 200), (32, 8, 128, 64, 4096),
                                                (24, 8, 128, 64, 3072)])
def test_gemm_skinny_qkv_rope_write(ops16, m, hq, hkv, hd, page, dim):
    """Projection + rotation + page write in one kernel, against the three separate kernels."""
    from fastgen_b200.cache import LayerMemory
    g = torch.Generator().manual_seed(m + hd)
    x = torch.randn(m, dim, generator=g).to(DEV, torch.bfloat16)
    w = (torch.randn((hq + 2 * hkv) * hd, dim, generator=g) / math.sqrt(dim)).to(DEV, torch.bfloat16)
    freqs = pl.rope_freqs(hd, 10000.0, None).to(DEV)
    n_pages, width = 40, 8
    table = torch.full((m + 1, width), -1, dtype=torch.int32)
    perm = torch.randperm(n_pages, generator=g).tolist()
    pos = torch.tensor([(7 * i + page - 1) % (page * width) for i in range(m)], dtype=torch.int32)
    req = torch.tensor([(i + 1) % (m + 1) for i in range(m)], dtype=torch.int32)
    req[m // 2] = -1 if m > 2 else req[m // 2]   # a padding lane
    for i in range(m):
        if req[i] >= 0:
            table[req[i], pos[i] // page] = perm.pop()
    mems = []
    for _ in range(2):
        kp = torch.zeros(n_pages, hkv, page, hd, dtype=torch.bfloat16, device=DEV)
        mems.append(LayerMemory(k_pages=kp, v_pages=torch.zeros_like(kp), block_table=table.to(DEV), page_size=page))
    pos, req = pos.to(DEV), req.to(DEV)
    from fastgen_b200.csrc import ops as O
    old, O.SKINNY_MAX_M = O.SKINNY_MAX_M, 32
    try:
        q = ops16.qkv_rope_write(x, w, pos, req, freqs, mems[0], hq, hkv, hd)
    finally:
        O.SKINNY_MAX_M = old
    assert q is not None
    qkv = ops16.linear(x, w)
    ops16.rope_kv_write(qkv[:, : hq * hd], qkv[:, hq * hd : (hq + hkv) * hd], qkv[:, (hq + hkv) * hd :], pos, req,
                        freqs, mems[1].k_pages, mems[1].v_pages, mems[1].block_table, page, hq, hkv, hd)
    ops16.check_status()
    live = (req >= 0).cpu()
    assert torch.allclose(q[live].float(), qkv[live][:, : hq * hd].float(), rtol=2e-2, atol=2e-2)
    assert torch.allclose(mems[0].k_pages.float(), mems[1].k_pages.float(), rtol=2e-2, atol=2e-2)
    assert torch.allclose(mems[0].v_pages.float(), mems[1].v_pages.float(), rtol=2e-2, atol=2e-2)
    assert torch.equal(mems[0].k_pages == 0, mems[1].k_pages == 0)   # the same slots were written, no others


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("ffn", [176, 331, 14336])
def test_silu_gate(ops32, dtype, ffn):
    g = torch.Generator().manual_seed(ffn)
    x = (torch.randn(11, 2 * ffn, generator=g) * 2).to(DEV, dtype)
    out = torch.empty(11, ffn, dtype=dtype, device=DEV)
    ops32.silu_gate(x, out)
    xd = x.double()
    ref = xd[:, :ffn] * torch.sigmoid(xd[:, :ffn]) * xd[:, ffn:]
    assert torch.allclose(out.double(), ref, **_tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hq,hkv,hd,page", [(4, 1, 16, 8), (6, 3, 32, 16), (5, 5, 48, 4), (32, 8, 128, 64)])
def test_rope_kv_write(ops32, dtype, hq, hkv, hd, page):
    g = torch.Generator().manual_seed(hd)
    t, n_pages, width = 23, 12, 6
    qkv = torch.randn(t, (hq + 2 * hkv) * hd, generator=g).to(DEV, dtype)
    orig = qkv.clone()
    freqs = pl.rope_freqs(hd, 10000.0, None).to(DEV)
    # two requests: slots 2 and 0; positions straddle page edges; one padding token
    req = torch.tensor([2] * 12 + [0] * 10 + [-1], dtype=torch.int32, device=DEV)
    pos = torch.tensor(list(range(page - 3, page + 9)) + list(range(0, 10)) + [5], dtype=torch.int32, device=DEV)
    table = torch.full((3, width), -1, dtype=torch.int32, device=DEV)
    perm = torch.randperm(n_pages, generator=g)
    table[2, :4] = perm[:4].to(DEV, torch.int32)
    table[0, :3] = perm[4:7].to(DEV, torch.int32)
    kp = torch.zeros(n_pages, hkv, page, hd, dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    q = qkv[:, : hq * hd]; k = qkv[:, hq * hd : (hq + hkv) * hd]; v = qkv[:, (hq + hkv) * hd :]
    ops32.rope_kv_write(q, k, v, pos, req, freqs, kp, vp, table, page, hq, hkv, hd)
    ops32.check_status()
    od = orig.double().cpu()
    rq = pl.apply_rope(od[:, : hq * hd].view(t, hq, hd), pos.cpu(), freqs.cpu()).view(t, -1)
    rk = pl.apply_rope(od[:, hq * hd : (hq + hkv) * hd].view(t, hkv, hd), pos.cpu(), freqs.cpu())
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    assert torch.allclose(q[:22].double().cpu(), rq[:22].cpu(), **tol)
    written = torch.zeros(n_pages, page, dtype=torch.bool)
    for i in range(22):
        pg = int(table[int(req[i]), int(pos[i]) // page]); off = int(pos[i]) % page
        written[pg, off] = True
        assert torch.allclose(kp[pg, :, off].double().cpu(), rk[i].cpu(), **tol)
        assert torch.equal(vp[pg, :, off].cpu(), orig[i, (hq + hkv) * hd :].view(hkv, hd).cpu())
    untouched = ~written
    assert torch.count_nonzero(kp.cpu().permute(0, 2, 1, 3)[untouched]) == 0
    # a position beyond the request's table is reported, not written
    pos2 = pos.clone(); pos2[0] = page * width + 1
    ops32.rope_kv_write(q, k, v, pos2, req, freqs, kp, vp, table, page, hq, hkv, hd)
    from fastgen_b200.csrc.ops import KernelError
    with pytest.raises(KernelError, match="block-table"):
        ops32.check_status()


# ---------------------------------------------------------------------------------
# attention: a step context by hand, a paged cache with shuffled pages
# ---------------------------------------------------------------------------------
def _attention_case(ops, seqs, hq, hkv, hd, page, window, seed, boost=None, use_tma=True, runs=1, layer=0,
                    pad_lanes=0):
    """seqs: list of (cached, new) per request.  Returns (out, ref) for the new tokens.
    ``runs``/``layer``: the pools hold ``runs`` layers (the others full of NaN) and the case
    lives in layer ``layer``.  ``pad_lanes``: that many single-token lanes of slot -1 are
    mixed in (a graph bucket larger than the step); their outputs are not compared."""
    from fastgen_b200.engine.step import StepContext

    dtype = ops.act_dtype
    g = torch.Generator().manual_seed(seed)
    total = [c + n for c, n in seqs]
    width = max(-(-t // page) for t in total) + 1
    n_pages = sum(-(-t // page) for t in total) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    kpool = torch.full((runs, n_pages, hkv, page, hd), float("nan"), dtype=dtype, device=DEV)
    vpool = torch.full((runs, n_pages, hkv, page, hd), float("nan"), dtype=dtype, device=DEV)
    kpool[layer] = torch.randn(n_pages, hkv, page, hd, generator=g).to(DEV, dtype)  # garbage in unused slots
    vpool[layer] = torch.randn(n_pages, hkv, page, hd, generator=g).to(DEV, dtype)
    kp, vp = kpool[layer], vpool[layer]
    table = torch.full((len(seqs) + 2, width), -1, dtype=torch.int32)
    ctx = StepContext(DEV)
    qs, refs, pos, req, keep = [], [], [], [], []
    slots = list(range(len(seqs) + 2))
    random.Random(seed).shuffle(slots)
    pad_after = set(random.Random(seed + 1).sample(range(len(seqs)), min(pad_lanes, len(seqs))))
    for b, (cached, new) in enumerate(seqs):
        slot = slots[b]
        t = cached + new
        k = torch.randn(t, hkv, hd, generator=g).to(dtype)
        v = torch.randn(t, hkv, hd, generator=g).to(dtype)
        q = torch.randn(t, hq, hd, generator=g).to(dtype)
        if boost is not None and t > boost[1]:
            # make one far key dominate one query: a fault in reaching it shows
            qi, kj = t - 1, boost[1]
            k[kj] = q[qi, 0 :: hq // hkv][:hkv] * 4.0
        for lp in range(-(-t // page)):
            pg = perm.pop()
            table[slot, lp] = pg
            rows = slice(lp * page, min(t, (lp + 1) * page))
            n = rows.stop - rows.start
            kp[pg, :, :n] = k[rows].permute(1, 0, 2).to(DEV)
            vp[pg, :, :n] = v[rows].permute(1, 0, 2).to(DEV)
        ref = pl.causal_attention(q.double(), k.double(), v.double(), hd ** -0.5, window)[cached:]
        refs.append(ref.reshape(new, hq * hd))
        qs.append(q[cached:].reshape(new, hq * hd))
        pos += list(range(cached, t)); req += [slot] * new; keep += [True] * new
        ctx.host_seq_slot.append(slot); ctx.host_seq_cached.append(cached)
        ctx.host_seq_start.append(ctx.host_seq_start[-1] + new)
        if b in pad_after:
            # a padding lane as a graph bucket has them: slot -1, position 0, some query
            qs.append(torch.randn(1, hq * hd, generator=g).to(dtype))
            pos.append(0); req.append(-1); keep.append(False)
            ctx.host_seq_slot.append(-1); ctx.host_seq_cached.append(0)
            ctx.host_seq_start.append(ctx.host_seq_start[-1] + 1)
    ctx.pos = torch.tensor(pos, dtype=torch.int32, device=DEV)
    ctx.req = torch.tensor(req, dtype=torch.int32, device=DEV)
    ctx.n_tokens = len(pos)
    q = torch.cat(qs).to(DEV)
    # queries live in a wider row, as in the fused projection
    wide = torch.zeros(q.shape[0], q.shape[1] + 2 * hkv * hd, dtype=dtype, device=DEV)
    wide[:, : q.shape[1]] = q
    out = torch.full((q.shape[0], hq * hd), float("nan"), dtype=dtype, device=DEV)
    from fastgen_b200.cache import LayerMemory
    mem = LayerMemory(k_pages=kp, v_pages=vp, block_table=table.to(DEV), page_size=page)
    if use_tma:
        mem.tensor_maps = ops.make_kv_tensor_maps(kpool, vpool, page)
        mem.layer_index = layer
    ops.attention(wide[:, : q.shape[1]], out, mem, ctx, hq, hkv, hd, window, hd ** -0.5)
    ops.check_status()
    keep = torch.tensor(keep)
    return out.double().cpu()[keep], torch.cat(refs)


CASES = [
    # (seqs, hq, hkv, hd, page, window)
    ([(0, 7), (0, 13), (0, 1), (0, 30)], 4, 1, 16, 8, None),
    ([(12, 1), (40, 9), (0, 70), (99, 1), (63, 2)], 6, 3, 32, 16, None),
    ([(5, 33), (90, 1), (64, 64), (23, 1)], 6, 2, 48, 8, 24),
    ([(300, 1), (0, 130), (255, 3), (128, 1)], 8, 2, 64, 64, None),
    ([(517, 1), (130, 70)], 32, 8, 128, 64, None),
    ([(127, 1), (128, 1), (129, 1), (0, 1)], 5, 5, 16, 4, 100),
    ([(200, 1), (10, 50)], 40, 2, 32, 16, None),   # a group of 20 heads
    ([(300, 1), (0, 1), (127, 1), (128, 1), (700, 1)], 8, 2, 64, 8, None),
    ([(1000, 1), (255, 1), (256, 1), (90, 1)], 6, 2, 128, 16, 300),
    ([(513, 1), (64, 1)], 16, 1, 128, 256, None),    # pages longer than a split
    ([(0, 300), (190, 75), (63, 2), (7, 130)], 8, 2, 64, 8, None),     # prompt portions, small pages
    ([(100, 200), (0, 129)], 6, 2, 128, 16, 90),                        # ... with a window
    ([(250, 260)], 4, 1, 128, 256, None),
    # enough (request, head, split) items for the persistent single-token kernel
    ([(900, 1), (130, 1), (767, 1), (768, 1), (5, 1), (640, 1), (899, 1), (0, 1), (127, 1), (128, 1), (511, 1),
      (333, 1)], 32, 8, 128, 64, None),
    ([(900, 1), (130, 1), (767, 1), (768, 1), (5, 1), (640, 1), (899, 1), (0, 1), (127, 1), (128, 1), (511, 1),
      (333, 1), (40, 30)], 16, 8, 128, 16, 300),
    ([(1500 + 37 * i, 1) for i in range(10)] + [(3 + 129 * i, 1) for i in range(10)], 20, 2, 64, 8, None),
    ([(1500, 1), (255, 1), (256, 1), (1023, 1), (1024, 1), (700, 1), (1, 1), (1300, 1)], 8, 8, 128, 256, None),
    # more (query tile, head) items than resident blocks: blocks of the prompt kernel take several items,
    # with odd and even numbers of key tiles each (the stages of their rings change sides between items)
    ([(37, 2600), (5, 1), (0, 70)], 16, 16, 64, 16, None),
]


@pytest.mark.parametrize("case", range(len(CASES)))
def test_attention(ops32, ops16, case):
    seqs, hq, hkv, hd, page, window = CASES[case]
    out, ref = _attention_case(ops32, seqs, hq, hkv, hd, page, window, case)
    assert torch.allclose(out, ref, rtol=1e-5, atol=1e-5), float((out - ref).abs().max())
    # tiled TMA loads where the shape allows (prompts on tcgen05 for head sizes 64 and 128,
    # then on mma.sync), else (and also) cp.async
    for use_tma, tc5 in ((True, True), (True, False), (False, False)):
        ops16.use_tcgen05 = tc5
        try:
            out, ref = _attention_case(ops16, seqs, hq, hkv, hd, page, window, case, use_tma=use_tma)
        finally:
            ops16.use_tcgen05 = True
        assert torch.allclose(out, ref, rtol=3e-2, atol=3e-2), (use_tma, tc5, float((out - ref).abs().max()))


@pytest.mark.parametrize("case", [3, 4, 8, 13, 14, 15, 16])
def test_attention_in_a_later_layer_with_padding_lanes(ops32, ops16, case):
    """The same cases in layer 2 of pools of 3 layers (the tiled loads' layer coordinate; the
    other layers hold NaN), with lanes of slot -1 among the single tokens."""
    seqs, hq, hkv, hd, page, window = CASES[case]
    pads = min(3, sum(1 for _, n in seqs if n == 1))
    out, ref = _attention_case(ops32, seqs, hq, hkv, hd, page, window, case, runs=3, layer=2, pad_lanes=pads)
    assert torch.allclose(out, ref, rtol=1e-5, atol=1e-5), float((out - ref).abs().max())
    for use_tma, tc5 in ((True, True), (True, False), (False, False)):
        ops16.use_tcgen05 = tc5
        try:
            out, ref = _attention_case(ops16, seqs, hq, hkv, hd, page, window, case, use_tma=use_tma, runs=3,
                                       layer=2, pad_lanes=pads)
        finally:
            ops16.use_tcgen05 = True
        assert torch.allclose(out, ref, rtol=3e-2, atol=3e-2), (use_tma, tc5, float((out - ref).abs().max()))


# One key among hundreds dominates the last query of every request (its score is 4 |q|^2 / sqrt(hd),
# tens of units above the rest): a kernel that misses that key, or sees it when a window hides
# it, is off by the size of a value, far beyond rounding.
SHARP_TOL = 6e-2


def _sharp(ops16, seqs, hq, hkv, hd, page, window, far, seed=77):
    for use_tma, tc5 in ((True, True), (True, False), (False, False)):
        ops16.use_tcgen05 = tc5
        try:
            out, ref = _attention_case(ops16, seqs, hq, hkv, hd, page, window, seed, boost=(None, far),
                                       use_tma=use_tma, runs=2, layer=1)
        finally:
            ops16.use_tcgen05 = True
        err = float((out - ref).abs().max())
        assert err < SHARP_TOL, (use_tma, tc5, far, err)


@pytest.mark.parametrize("hd,hq,hkv", [(64, 8, 2), (128, 8, 2), (128, 24, 2)])
@pytest.mark.parametrize("page", [16, 64, 256])
def test_attention_reaches_a_far_key_tiled(ops16, hd, hq, hkv, page):
    """At the head sizes of the tiled-load kernels (tcgen05 and mma.sync prompts, the persistent and
    the one-block-a-split single-token kernels; 24 heads over 2 is a group of 12, which the persistent
    kernel does not take), the dominant key lies at 0, at the ends of key tiles, of splits and of pages."""
    fars = sorted({0, 63, 64, 127, 128, page - 1, page, 2 * page - 1, 255, 256, 383})
    singles = [(399 + i, 1) for i in range(13)]   # 13 requests: the persistent kernel where the group allows
    for far in fars:
        _sharp(ops16, [(0, 400)], hq, hkv, hd, page, None, far)
        _sharp(ops16, [(250, 150)], hq, hkv, hd, page, None, far)
        _sharp(ops16, singles, hq, hkv, hd, page, None, far)


@pytest.mark.parametrize("hd,hq,hkv", [(64, 8, 2), (128, 4, 1), (128, 12, 1)])
@pytest.mark.parametrize("page", [16, 64])
def test_attention_window_edge_tiled(ops16, hd, hq, hkv, page):
    """The key at pos - window must be out, the one at pos - window + 1 in: prompts (60, 40) and
    (250, 150), single tokens alone and a dozen together."""
    for window in (24, 100, 129):
        for seqs in ([(60, 40)], [(250, 150)], [(399, 1)], [(399, 1)] * 12):
            last = seqs[0][0] + seqs[0][1] - 1
            for far in (last - window, last - window + 1):
                if far >= 0:
                    _sharp(ops16, seqs, hq, hkv, hd, page, window, far, seed=5)


@pytest.mark.parametrize("hd,hq,hkv,page", [(128, 8, 2, 64), (64, 6, 2, 16), (128, 4, 1, 256), (64, 24, 2, 64)])
def test_attention_long_items_in_parts(ops16, hd, hq, hkv, page):
    """A launch of few (query tile, head) items works on an item of 16 key tiles or more in several
    parts and adds them up in a second kernel.  The dominant key lies at the first and last key of
    the parts (with 2,040 keys and 8 tiles a part: 512 keys each), the other requests of the call
    are long, short (not split) and of few tokens; with a window the parts start at its edge."""

    def parts_seen():
        # the kernel leaves the number of parts of every item of its last launch
        if hd not in ops16._split:
            return set()
        flags = ops16._split[hd][1]
        assert int(flags[0::2].abs().max()) == 0  # the counters are back at zero
        seen = set(flags[1::2].tolist()) - {0}
        flags.zero_()
        return seen

    parts_seen()  # (forget what earlier tests left)
    for far in (0, 511, 512, 1023, 1024, 1535, 1536, 2039):
        _sharp(ops16, [(2000, 40)], hq, hkv, hd, page, None, far)
    assert parts_seen() == {4}  # 32 key tiles: four parts of 8
    for far in (0, 700, 1472, 2700, 3008):
        _sharp(ops16, [(1500, 100), (3000, 9), (100, 30)], hq, hkv, hd, page, None, far)
    assert parts_seen() == {3, 6}  # 25 and 48 key tiles; the short request's items are not split
    for far in (3008 - 1100, 3008 - 1100 + 1, 2500):
        _sharp(ops16, [(3000, 9), (1200, 2)], hq, hkv, hd, page, 1100, far, seed=5)
    assert parts_seen() == {2}  # 19 and 18 key tiles from the window's edge on
    # random values, against the plain reference under the rule of the other cases
    out, ref = _attention_case(ops16, [(4000, 70), (1000, 3)], hq, hkv, hd, page, None, seed=3, runs=2, layer=1)
    assert float((out - ref).abs().max()) < 2e-2
    parts_seen()
    # 97 key tiles for up to 16 parts of at least 8: 12 parts of 9 tiles would leave the last one empty
    out, ref = _attention_case(ops16, [(6145, 60)], hq, hkv, hd, page, None, seed=4, runs=2, layer=1)
    assert float((out - ref).abs().max()) < 2e-2
    assert parts_seen() == {11}


@pytest.mark.parametrize("far", [0, 63, 64, 127, 128, 300])
def test_attention_reaches_a_far_key(ops32, ops16, far):
    """One key among hundreds dominates the last query: it must be found wherever it lies."""
    for ops, tol in ((ops32, 1e-4), (ops16, 5e-2)):
        for seqs in ([(0, 400)], [(399, 1)], [(250, 150)]):
            out, ref = _attention_case(ops, seqs, 4, 2, 32, 16, None, 77, boost=(None, far))
            assert float((out - ref).abs().max()) < tol


def test_attention_window_edge(ops32, ops16):
    """The key at pos - window must be out, the one at pos - window + 1 in."""
    for ops, tol in ((ops32, 1e-4), (ops16, 5e-2)):
        for far in (75, 76):  # last query at 99, window 24: keys 76..99 are visible
            out, ref = _attention_case(ops, [(99, 1)], 2, 1, 16, 8, 24, 5, boost=(None, far))
            assert float((out - ref).abs().max()) < tol
            out, ref = _attention_case(ops, [(60, 40)], 2, 1, 16, 8, 24, 5, boost=(None, far))
            assert float((out - ref).abs().max()) < tol


def test_attention_missing_page_is_reported(ops16):
    from fastgen_b200.csrc.ops import KernelError
    from fastgen_b200.engine.step import StepContext
    ctx = StepContext(DEV)
    ctx.host_seq_slot, ctx.host_seq_cached, ctx.host_seq_start = [0], [20], [0, 1]
    ctx.pos = torch.tensor([20], dtype=torch.int32, device=DEV)
    ctx.req = torch.tensor([0], dtype=torch.int32, device=DEV)
    table = torch.tensor([[0, -1, 2]], dtype=torch.int32, device=DEV)  # page of positions 8..15 is missing
    from fastgen_b200.cache import LayerMemory
    for hd in (16, 64):  # the cp.async kernel and the TMA kernel
        kp = torch.zeros(3, 1, 8, hd, dtype=torch.bfloat16, device=DEV)
        q = torch.zeros(1, hd, dtype=torch.bfloat16, device=DEV)
        out = torch.empty_like(q)
        mem = LayerMemory(k_pages=kp, v_pages=kp, block_table=table, page_size=8,
                          tensor_maps=ops16.make_kv_tensor_maps(kp[None], kp[None], 8))
        assert (mem.tensor_maps is not None) == (hd == 64)
        ops16.attention(q, out, mem, ctx, 1, 1, hd, None, 0.25)
        with pytest.raises(KernelError, match="block-table"):
            ops16.check_status()


def test_a_wait_that_runs_out_is_reported(ops16):
    """The bounded wait of the kernels on a barrier nobody arrives at (a short limit): it
    returns, the status word says so, the block's other waits are released at once, and a
    wait on a completed phase is untouched."""
    from fastgen_b200.csrc.ops import KernelError
    first, second, cycles_first, cycles_second, completed = ops16.wait_timeout_selftest(limit=4096)
    assert first == 0 and second == 0 and completed == 1
    assert 0 < cycles_second < cycles_first / 8, (cycles_first, cycles_second)
    with pytest.raises(KernelError, match="a bounded wait inside a kernel gave up"):
        ops16.check_status()
    ops16.check_status()  # the word is clear again


# ---------------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------------
def test_argmax_and_logprobs(ops32):
    g = torch.Generator().manual_seed(1)
    for vocab in (5, 331, 128256):
        logits = torch.randn(7, vocab, generator=g).to(DEV)
        logits[2, vocab // 2] = logits[2, vocab - 1] = 9.0  # a tie: the lowest index wins
        out = torch.empty(7, dtype=torch.int32, device=DEV)
        lp = torch.empty(7, dtype=torch.float32, device=DEV)
        ops32.sample(logits, None, 1.0, 0, None, None, out, lp, None)
        # the status word rides along when asked for
        out1 = torch.full((8,), -5, dtype=torch.int32, device=DEV)
        ops32.status.fill_(6)
        ops32.sample(logits, None, 1.0, 0, None, None, out1, None, None, with_status=True)
        ops32.status.zero_()
        assert torch.equal(out1[:7], out) and int(out1[7]) == 6
        ref = logits.argmax(-1)
        assert out[2] == vocab // 2
        keep = [0, 1, 3, 4, 5, 6]
        assert torch.equal(out[keep].long(), ref[keep])
        ref_lp = torch.log_softmax(logits.double(), -1)[torch.arange(7), out.long()]
        assert torch.allclose(lp.double(), ref_lp, atol=1e-4)


@pytest.mark.parametrize("top_p", [1.0, 0.9, 0.5])
def test_sampling_matches_inverse_cdf(ops32, top_p):
    g = torch.Generator().manual_seed(2)
    rows, vocab = 64, 1000
    logits = (torch.randn(rows, vocab, generator=g) * 2).to(DEV)
    temps = torch.full((rows,), 0.8, device=DEV)
    keys = torch.arange(rows, dtype=torch.int64, device=DEV)
    posn = torch.arange(100, 100 + rows, dtype=torch.int32, device=DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    scratch = torch.empty(rows * vocab, device=DEV)
    ops32.sample(logits, temps, top_p, 1234, keys, posn, out, None, scratch)
    u = ops32.sample_uniform(1234, keys, posn).double().cpu()
    assert 0 <= u.min() and u.max() < 1
    probs = pl.softmax_temperature(logits.cpu(), 0.8)
    keep = pl.top_p_keep(probs, top_p) if top_p < 1 else torch.ones_like(probs, dtype=torch.bool)
    kept = torch.where(keep, probs, torch.zeros_like(probs))
    cdf = torch.cumsum(kept, -1)
    exact = 0
    for r in range(rows):
        tok = int(out[r])
        assert keep[r, tok], "a token outside the nucleus was drawn"
        goal = u[r] * cdf[r, -1]
        lo = cdf[r, tok] - kept[r, tok]
        # the drawn token's interval contains u * mass, up to float32 rounding of the sums
        assert lo - 1e-4 <= goal <= cdf[r, tok] + 1e-4
        exact += int(torch.searchsorted(cdf[r], goal, right=True)) == tok
    assert exact >= rows - 2
    # the same keys give the same tokens whatever the batch; other keys give others
    out2 = torch.empty(8, dtype=torch.int32, device=DEV)
    ops32.sample(logits[8:16].contiguous(), temps[:8], top_p, 1234, keys[8:16].contiguous(),
                 posn[8:16].contiguous(), out2, None, scratch)
    assert torch.equal(out2, out[8:16])


def test_sampling_distribution(ops32):
    vocab, rows = 16, 4096
    logits = torch.linspace(-2, 2, vocab).repeat(rows, 1).to(DEV)
    temps = torch.ones(rows, device=DEV)
    keys = torch.arange(rows, dtype=torch.int64, device=DEV)
    posn = torch.zeros(rows, dtype=torch.int32, device=DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops32.sample(logits, temps, 1.0, 99, keys, posn, out, None, torch.empty(rows * vocab, device=DEV))
    freq = torch.bincount(out.long().cpu(), minlength=vocab).double() / rows
    probs = torch.softmax(torch.linspace(-2, 2, vocab).double(), 0)
    assert float((freq - probs).abs().max()) < 0.02
    u = ops32.sample_uniform(99, keys, posn).cpu()
    assert abs(float(u.mean()) - 0.5) < 0.02 and abs(float(u.var()) - 1 / 12) < 0.01

