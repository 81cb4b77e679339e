"""Time the bfloat16 attention kernels alone, on a cache filled with random values.

    python -m fastgen_b200.tools.attention_bench                      # a table of prompt and single-token shapes
    python -m fastgen_b200.tools.attention_bench --prompt 2048,0 --prompt 8192,32768 --single 8,4096

``--prompt T,C``: one request that brings T tokens on C cached positions (the prompt kernel);
``--single B,C``: B requests that bring one token each on C cached positions (the split
kernel and the merge of its splits).  Times are CUDA-event times of back-to-back launches
after a warm-up; keys and values of a prompt case mostly come from L2, as they do in a step,
where the kernel before has just written them.  Prompt cases report TFLOP/s (causal: 4 hd
heads (T C + T (T + 1) / 2)), single-token cases the GB/s of keys and values they must read.
"""

from __future__ import annotations

import argparse


def _context(ops, torch, seqs, hq, hkv, hd, page):
    """A step context and a cache for ``seqs`` = [(cached, new)], pages in order."""
    from ..cache import LayerMemory
    from ..engine.step import StepContext

    dev = ops.device
    pages_of = [-(-(c + n) // page) for c, n in seqs]
    n_pages = sum(pages_of) + 2
    kp = torch.randn(1, n_pages, hkv, page, hd, device=dev, dtype=torch.bfloat16)
    vp = torch.randn(1, n_pages, hkv, page, hd, device=dev, dtype=torch.bfloat16)
    table = torch.full((len(seqs), max(pages_of)), -1, dtype=torch.int32)
    ctx = StepContext(dev)
    pos, req, first = [], [], 0
    for b, (cached, new) in enumerate(seqs):
        table[b, : pages_of[b]] = torch.arange(first, first + pages_of[b], dtype=torch.int32)
        first += pages_of[b]
        pos += list(range(cached, cached + new))
        req += [b] * new
        ctx.host_seq_slot.append(b)
        ctx.host_seq_cached.append(cached)
        ctx.host_seq_start.append(ctx.host_seq_start[-1] + new)
    ctx.pos = torch.tensor(pos, dtype=torch.int32, device=dev)
    ctx.req = torch.tensor(req, dtype=torch.int32, device=dev)
    ctx.n_tokens = len(pos)
    mem = LayerMemory(k_pages=kp[0], v_pages=vp[0], block_table=table.to(dev), page_size=page)
    mem.tensor_maps = ops.make_kv_tensor_maps(kp, vp, page)
    return ctx, mem, (kp, vp)


def time_case(ops, torch, seqs, hq, hkv, hd, page, reps: int = 20) -> float:
    """Microseconds of one attention call for the step ``seqs``."""
    ctx, mem, _keep = _context(ops, torch, seqs, hq, hkv, hd, page)
    q = torch.randn(ctx.n_tokens, hq * hd, device=ops.device, dtype=torch.bfloat16)
    out = torch.empty_like(q)

    def call():
        ops.attention(q, out, mem, ctx, hq, hkv, hd, None, hd ** -0.5)

    for _ in range(3):
        call()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        call()
    b.record()
    torch.cuda.synchronize()
    ops.check_status()
    return a.elapsed_time(b) / reps * 1e3


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--prompt", action="append", default=[], metavar="T,C")
    ap.add_argument("--single", action="append", default=[], metavar="B,C")
    ap.add_argument("--heads", default="32,8", help="query heads, key/value heads")
    ap.add_argument("--head-dim", type=int, action="append", default=[])
    ap.add_argument("--page", type=int, default=64)
    args = ap.parse_args(argv)

    import torch

    from ..csrc.ops import Ops

    ops = Ops(torch.bfloat16, "cuda:0")
    hq, hkv = (int(x) for x in args.heads.split(","))
    prompts = [tuple(int(x) for x in p.split(",")) for p in args.prompt]
    singles = [tuple(int(x) for x in s.split(",")) for s in args.single]
    if not prompts and not singles:
        prompts = [(512, 0), (2048, 0), (8192, 0), (2048, 8192), (512, 16384), (8192, 32768), (256, 32768), (64, 32768),
                   (8, 32768)]
        singles = [(1, 4096), (8, 4096), (64, 4096), (1, 65536), (8, 65536)]
    for hd in args.head_dim or [128, 64]:
        for t, cached in prompts:
            us = time_case(ops, torch, [(cached, t)], hq, hkv, hd, args.page)
            flops = 4 * hd * hq * (t * cached + t * (t + 1) / 2)
            print(f"head size {hd}, prompt of {t} on {cached} cached: {us:9.1f} us  {flops / us / 1e6:7.1f} TFLOP/s",
                  flush=True)
        for batch, cached in singles:
            us = time_case(ops, torch, [(cached, 1)] * batch, hq, hkv, hd, args.page)
            read = batch * (cached + 1) * 2 * hkv * hd * 2
            print(f"head size {hd}, {batch} single tokens on {cached} cached: {us:9.1f} us  {read / us / 1e3:7.1f} GB/s",
                  flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
