#!/usr/bin/env python3
"""Benchmark: decode tokens/s and prefill tokens/s of a Llama-3.1-8B-shaped model.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step.  The default run has the layer sizes of Llama 3.1 8B
with random weights, a batch of 8 and a context of 4,096 tokens: the timed
steps end at position 4,096.  One JSON line is printed (see the keys below).
"""

from __future__ import annotations

import argparse
import json
import os
import queue
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LLAMA_8B = dict(
    architectures=["LlamaForCausalLM"], hidden_size=4096, intermediate_size=14336,
    num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, rms_norm_eps=1e-5,
    vocab_size=128256, tie_word_embeddings=False, rope_theta=500000.0,
    rope_scaling=dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192, rope_type="llama3"),
    max_position_embeddings=131072,
)
# the layer sizes of Llama 3.2 1B / 3B (BASELINE.json configs 4 and 3), for --shape
SHAPES = {
    "8b": LLAMA_8B,
    "3b": dict(LLAMA_8B, hidden_size=3072, intermediate_size=8192, num_hidden_layers=28, num_attention_heads=24,
               num_key_value_heads=8, tie_word_embeddings=True,
               rope_scaling=dict(LLAMA_8B["rope_scaling"], factor=32.0)),
    "1b": dict(LLAMA_8B, hidden_size=2048, intermediate_size=8192, num_hidden_layers=16, num_attention_heads=32,
               num_key_value_heads=8, tie_word_embeddings=True,
               rope_scaling=dict(LLAMA_8B["rope_scaling"], factor=32.0)),
}
PAGE = 64
SEED = 4
PREFILL_TOKENS = 2048
SETTLE_S = 0.5  # pause between filling the cache and the decode steps


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        p = json.loads(path.read_text())
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.proc = None
        self.lines = []

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for name, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=mx, reasons=sorted(reasons),
                    samples=len(sm))


def model_flops(cfg: dict, n_layers: int, t: int, rows: int, cached: int = 0) -> float:
    """FLOPs of a step of t prompt tokens on `cached` keys with logits at `rows` places."""
    d, f, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hq, hkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = d // hq
    per_layer = 2 * t * d * (hq + 2 * hkv) * hd + 2 * t * hq * hd * d + 3 * 2 * t * d * f
    attn = 4 * hd * hq * (t * cached + t * (t + 1) / 2)
    return n_layers * (per_layer + attn) + 2 * rows * d * v


def describe_config(cfg: dict, batch: int, context: int, layers: int, layers_full: int, first: int, last: int,
                    peaks_source: str, shape: str = "8b") -> dict:
    """The sizes of the run, flat (the record keeps at most 20 keys of it, and no lists)."""
    name = {"8b": "Llama-3.1-8B shape", "3b": "Llama-3.2-3B shape", "1b": "Llama-3.2-1B shape"}[shape]
    return {
        "model": name, "global_batch": batch, "seq_len": context,
        "parallelism": "single GPU", "layers": layers, "layers_full": layers_full,
        "hidden": cfg["hidden_size"], "ffn": cfg["intermediate_size"], "q_heads": cfg["num_attention_heads"],
        "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["hidden_size"] // cfg["num_attention_heads"],
        "vocab": cfg["vocab_size"], "page": PAGE, "decode_from": first, "decode_to": last,
        "prefill_tokens": PREFILL_TOKENS, "settle_s": SETTLE_S,
        "l2": "inputs larger than L2 (all weights are streamed every step)", "peaks": peaks_source,
    }


def run_ours(args) -> dict:
    import torch

    from fastgen_b200.config import model_args_from_config
    from fastgen_b200.csrc.ops import Ops
    from fastgen_b200.engine import Engine, Fastgen, GenArgs, Model, Packet, StepEntry
    from fastgen_b200.sampling import Sampler

    pk = peaks()
    cfg = dict(SHAPES[args.shape])
    full_layers = cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = args.layers or full_layers
    n_layers = cfg["num_hidden_layers"]
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    margs = model_args_from_config(cfg)
    model = Model.random(margs, torch.bfloat16, dev, seed=SEED)
    vocab = cfg["vocab_size"]
    ctx_len = args.context
    k, w = args.steps, args.warmup
    # the timed steps end at the context length, or (--from-position) start at that position
    prompt_len = max(1, (args.from_position if args.from_position else ctx_len - k) - w)
    max_b = max(args.batch, 64 if not args.skip_points else args.batch, 1)
    n_pages = max_b * (-(-(ctx_len + 1) // PAGE)) + PREFILL_TOKENS // PAGE + 2
    longest = max(ctx_len, PREFILL_TOKENS)
    if args.more_points:
        # room for 8 requests of 65,536 tokens and for a portion of 8,192 on 32,768 cached keys
        n_pages = max(n_pages, 8 * (65536 // PAGE + 1) + 8)
        longest = max(longest, 65536)
    engine = Engine(model, page_size=PAGE, n_pages=n_pages, max_requests=max_b,
                    max_length=longest + PAGE, num_cuda_graphs=max_b,
                    # prompt steps replay CUDA graphs of their padded shape, as in the generator
                    max_step_tokens=8192 if args.more_points else PREFILL_TOKENS)
    sampler = Sampler(model.ops, vocab, max_b, use_sampling=False)
    gen = torch.Generator().manual_seed(SEED)

    def prompt(n):
        return torch.randint(0, vocab, (n,), generator=gen).tolist()

    def event_ms(fn, reps):
        times = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        return times

    # ---- prefill of 2,048 tokens (one whole prompt, logits at its last token) ----
    toks = prompt(PREFILL_TOKENS)

    def prefill_once():
        engine.admit("p")
        engine.step([StepEntry("p", toks, [PREFILL_TOKENS - 1])])
        engine.release("p")

    pre_ms = float("nan")
    if not args.skip_prefill:
        for _ in range(3):
            prefill_once()
        pre_ms = min(event_ms(prefill_once, 5))
    pre_flops = model_flops(cfg, n_layers, PREFILL_TOKENS, 1)
    prefill = None if args.skip_prefill else dict(value=round(PREFILL_TOKENS / pre_ms * 1e3, 1), tokens=PREFILL_TOKENS, ms=round(pre_ms, 3),
                   frac=round(pre_flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                   tflops=round(pre_flops / (pre_ms * 1e-3) / 1e12, 1), peak_tflops=pk["bf16_tflops"])

    # ---- decode, device-timed: K graph replays + sampling, tokens stay on the device ----
    filled = []  # (profiling and the far points: the cache pages hold random values instead of real keys)
    weight_bytes = model.weight_bytes()  # every matrix once; the embedding table only if it is the output
    kv_per_token = model.cache_bytes_per_token(2)

    def decode_run(batch, steps, warm, clocks=None, prompt_len=prompt_len, fast_fill=args.fast_fill):
        ids = [f"d{i}" for i in range(batch)]
        for rid in ids:
            engine.admit(rid)
        for rid in ids:  # fill the cache: the prompt in portions of 2,048
            if fast_fill:
                r = engine.cache.get(rid)
                engine.cache.reserve(r, prompt_len)
                engine.cache.advance(r, prompt_len)
                continue
            p = prompt(prompt_len)
            for s in range(0, prompt_len, PREFILL_TOKENS):
                engine.step([StepEntry(rid, p[s:s + PREFILL_TOKENS], [])])
        if fast_fill and not filled:
            for grp in engine.cache.groups:
                grp.k_pages.normal_(0.0, 1.0)
                grp.v_pages.normal_(0.0, 1.0)
            filled.append(True)
        reqs = [engine.cache.get(rid) for rid in ids]
        slots = [r.slot for r in reqs]
        tokens = torch.randint(0, vocab, (batch,), generator=gen).to(dev, torch.int32)
        launches0 = None

        def one_step():
            nonlocal tokens
            for r in reqs:
                engine.cache.reserve(r, r.length + 1)
            engine.cache.flush_tables()
            logits = engine.graphs.run(tokens, [r.length for r in reqs], slots)
            tokens, _ = sampler.sample(logits, [0.0] * batch, [0] * batch, [0] * batch)
            for r in reqs:
                engine.cache.advance(r, r.length + 1)

        # the prompts' prefill has just run at the power cap: let the clocks settle before the
        # decode steps are warmed up and timed (nothing runs meanwhile)
        torch.cuda.synchronize()
        time.sleep(SETTLE_S)
        for _ in range(warm):
            one_step()
        torch.cuda.synchronize()
        if clocks:
            clocks.start()
        launches0 = Ops.launches
        first_len = reqs[0].length
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            one_step()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        launches = Ops.launches - launches0
        last_len = reqs[0].length
        engine.ops.check_status()
        for rid in ids:
            engine.release(rid)
        avg_ctx = (first_len + last_len) / 2
        step_bytes = weight_bytes + batch * avg_ctx * kv_per_token
        return dict(ms_per_step=ms / steps, tok_s=batch * steps / ms * 1e3, launches=launches,
                    gbs=step_bytes / (ms / steps * 1e-3) / 1e9, first=first_len, last=last_len)

    if args.skip_decode:
        print(json.dumps({"impl": "ours", "prefill": prefill, "note": "decode skipped"}))
        sys.exit(0)
    clocks = ClockSampler()
    main = decode_run(args.batch, k, w, clocks)
    # ---- the same through the Python entry point: host tokens in, host tokens out ----
    # As the reference arm measures itself (baseline/reference_arm.py): the same prompts are
    # generated twice, for `warmup` and for `warmup + n` new tokens, all prompts admitted and
    # prefilled in one step, and the difference of the wall-clock times is divided into the
    # difference of the generated tokens.  n is at least 200 decode steps of the full batch; every
    # step's tokens come from pinned host memory and its sampled tokens are read back to the host.
    e2e = None
    if not args.skip_e2e:
        n_e2e = max(k, 200)
        e2e_prompt = max(1, ctx_len - n_e2e - w)
        fg = Fastgen(GenArgs(use_sampling=False, max_batch=args.batch, max_seq=args.batch * (ctx_len + PAGE),
                             cache_block=PAGE, max_prefill=args.batch * ctx_len, num_cuda_graphs=args.batch),
                     model, stop_tokens=[])
        prompts = [prompt(e2e_prompt) for _ in range(args.batch)]

        def generate(max_gen):
            q = queue.Queue()
            for i, p in enumerate(prompts):
                q.put(Packet(thread_id=i, tokens=p, max_gen=max_gen))
            q.put(None)
            first = len(fg.step_log)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            n = sum(len(p.tokens) for p in fg.generate(q))
            torch.cuda.synchronize()
            return time.perf_counter() - t0, n, fg.step_log[first:]

        generate(2)
        t_short, n_short, _ = generate(w)
        t_long, n_long, log = generate(w + n_e2e)
        full = [s for s in log if s["prompt_tokens"] == 0 and s["decode_tokens"] == args.batch]
        e2e = dict(value=round((n_long - n_short) / (t_long - t_short), 1), unit="tokens/s",
                   h2d_bytes_per_step=int(sum(s["h2d_bytes"] for s in full) / max(1, len(full))),
                   d2h_bytes_per_step=int(sum(s["d2h_bytes"] for s in full) / max(1, len(full))),
                   steps=n_e2e, generated=n_long, full_batch_steps=len(full),
                   wall_s=round(t_long - t_short, 4), host_sync_every_steps=fg.gen_args.sync_freq,
                   method="wall clock of generate(): (tokens B - tokens A) / (time B - time A)")
        fg.destroy()
    clk = clocks.stop()

    # ---- the other batch sizes (after the end-to-end run, which shares the main run's conditions) ----
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            r = decode_run(b, min(k, 128), w)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            points[f"decode_b{b}_hbm_frac"] = round(r["gbs"] / pk["hbm_gbs"], 4)
    points[f"decode_b{args.batch}"] = round(main["tok_s"], 1)
    if args.more_points:
        # Further sizes: decode at contexts of 16,384 and 65,536 (the pages hold random values: a
        # decode step's time does not depend on them), and prompt portions of 512 and 8,192 tokens
        # on 8,192 and 32,768 cached keys.  Each with its fraction of the roofline.
        for ctx in (16384, 65536):
            for b in (1, 8):
                r = decode_run(b, 64, w, prompt_len=ctx - 64 - w, fast_fill=True)
                points[f"decode_b{b}_ctx{ctx // 1024}k"] = round(r["tok_s"], 1)
                points[f"decode_b{b}_ctx{ctx // 1024}k_hbm_frac"] = round(r["gbs"] / pk["hbm_gbs"], 4)
        for t, cached in ((512, 8192), (8192, 8192), (512, 32768), (8192, 32768), (8192, 0)):
            portion = prompt(t)

            def portion_once():
                engine.admit("far")
                r = engine.cache.get("far")
                if cached:
                    engine.cache.reserve(r, cached)
                    engine.cache.advance(r, cached)
                engine.step([StepEntry("far", portion, [t - 1])])
                engine.release("far")

            if not filled:
                for grp in engine.cache.groups:
                    grp.k_pages.normal_(0.0, 1.0)
                    grp.v_pages.normal_(0.0, 1.0)
                filled.append(True)
            portion_once()
            ms = min(event_ms(portion_once, 3))
            flops = model_flops(cfg, n_layers, t, 1, cached)
            key = f"prefill_t{t}_on{cached // 1024}k"
            points[key] = round(t / ms * 1e3, 1)
            points[key + "_tensor_frac"] = round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)

    return {
        "metric": f"decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens ({args.shape.upper()}, bf16)",
        "value": round(main["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": k, "warmup": w,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights seed 4, uniform random token ids)",
        "impl": "ours",
        "config": describe_config(cfg, args.batch, ctx_len, n_layers, full_layers, main["first"], main["last"],
                                  pk["source"], args.shape),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(main["gbs"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(main["gbs"] / pk["hbm_gbs"], 4)},
        "points": points,
        "e2e": e2e,
        "gpu_launches": main["launches"],
        "clocks": clk,
    }


def run_reference(args) -> dict:
    sys.path.insert(0, str(ROOT / "baseline"))
    try:
        from reference_arm import run
    except Exception as e:  # the arm's own module is missing or broken
        return {"impl": "reference", "unavailable": f"reference arm not runnable: {e!r}"[:300]}
    return run(args, SHAPES[args.shape])


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None,
                    help="timed decode steps (default 256, or up to the context length with --from-position)")
    ap.add_argument("--from-position", type=int, default=0,
                    help="time the decode steps from this position on (e.g. 2048, with --context 4096: the "
                         "steps span 2,048 -> 4,096); default: the steps end at the context length")
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0: all)")
    ap.add_argument("--shape", choices=sorted(SHAPES), default="8b",
                    help="layer sizes: Llama 3.1 8B (the benchmark's), Llama 3.2 3B or 1B")
    ap.add_argument("--skip-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--more-points", action="store_true",
                    help="also measure decode at contexts of 16k and 64k and prompt portions on 8k and 32k cached keys")
    ap.add_argument("--skip-prefill", action="store_true", help="skip the 2,048-token prefill measurement")
    ap.add_argument("--skip-e2e", action="store_true", help="skip the run through the Python entry point")
    ap.add_argument("--skip-decode", action="store_true", help="skip the decode measurement (profiling prefill)")
    ap.add_argument("--fast-fill", action="store_true",
                    help="profiling only: fill the cache pages with random values instead of prefilling the prompts")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.from_position and not 0 < args.from_position < args.context:
        ap.error("--from-position must lie inside the context")
    if args.steps is None:
        args.steps = args.context - args.from_position if args.from_position else 256
    if args.from_position and args.from_position + args.steps > args.context:
        ap.error("--from-position + --steps goes beyond --context")
    out = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
