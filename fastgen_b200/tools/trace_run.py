"""Trace replay: feed given token ids through the engine and write logits."""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path



def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__)
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder the logits are written to")
    parser.add_argument(
        "--max-tokens", type=int, required=True,
        help="most tokens live requests hold at any time (each rounded up to whole pages)",
    )
    parser.add_argument("--page-size", type=int, default=64, help="tokens per cache page")
    parser.add_argument("--max-requests", type=int, default=4, help="most requests live at a time")
    parser.add_argument("--device", default="cuda:0")
    args = parser.parse_args(argv)

    import torch

    from ..engine import Engine, Model, StepEntry

    if args.page_size <= 0:
        parser.error("--page-size must be positive")
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)

    model = Model.load(args.model, dtype, args.device)
    # --max-tokens counts every live request rounded up to a multiple of 64; pages that do
    # not divide 64 (larger ones above all) may need up to one page more a live request
    slack = 0 if 64 % args.page_size == 0 else args.max_requests * args.page_size
    n_pages = max(1, -(-(args.max_tokens + slack) // args.page_size))
    engine = Engine(
        model,
        page_size=args.page_size,
        n_pages=n_pages,
        max_requests=args.max_requests,
        max_length=min(model.args.max_positions, n_pages * args.page_size),
    )
    live = set()
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            if e["id"] not in live:
                engine.admit(e["id"])
                live.add(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e.get("want", [])))
        logits = engine.step(entries)
        if logits is not None:
            arr = logits.detach().to("cpu", torch.float32).numpy().astype("<f4", copy=False)
            arr.tofile(out_dir / f"{step}.f32")
        else:
            torch.cuda.synchronize()
        engine.ops.check_status()
        for rid in rec.get("end", []):
            if rid in live:
                engine.release(rid)
                live.discard(rid)
        print(f"done {step}", flush=True)
    return 0
