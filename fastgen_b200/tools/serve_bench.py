"""Throughput of continuous batching through the Python entry point.

Many requests of different lengths go through ``Fastgen.generate`` at once: the
scheduler admits them as pages allow, cuts prompts into portions under the token
budget beside the decoding requests, and frees what finishes.  Weights are random
(seeded), token ids uniform random; no request stops before its length limit.

    python -m fastgen_b200.tools.serve_bench --shape 3b     # 64 requests, prompts U[128, 2048], 256 new tokens
    python -m fastgen_b200.tools.serve_bench --shape 1b     # 256 requests, prompts U[16, 1024], U[32, 512] new tokens,
                                                            # arriving one after another over --arrive-over seconds

The shapes are those of Llama 3.2 1B / 3B and Llama 3.1 8B (layer sizes only; the
weights are random).  One JSON line is printed: generated tokens a second over the
whole run (wall clock around ``generate``, host tokens in and out), prompt tokens a
second, steps, preemptions, and what the steps achieved against the roofline: for
the steps of decoded tokens only, the bytes they had to read (every weight once and
the cached keys and values of their requests) over their time, as a fraction of the
HBM bandwidth; for the steps that are mostly prompt portions, their FLOPs over their
time as a fraction of the tensor-core peak; and the share of steps in which prompt
portions and decoded tokens ran side by side.

With ``--arrive-over S`` (the 1B workload's default: 1.0) a producer thread puts the
requests into the generator's queue on a seeded schedule (exponential gaps, scaled to span
S seconds), so requests keep arriving while others decode.
"""

from __future__ import annotations

import argparse
import json
import queue
import random
import threading
import time
from pathlib import Path

SHAPES = {
    "1b": dict(hidden_size=2048, intermediate_size=8192, num_hidden_layers=16, num_attention_heads=32,
               num_key_value_heads=8, head_dim=64, tie_word_embeddings=True, factor=32.0),
    "3b": dict(hidden_size=3072, intermediate_size=8192, num_hidden_layers=28, num_attention_heads=24,
               num_key_value_heads=8, head_dim=128, tie_word_embeddings=True, factor=32.0),
    "8b": dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, tie_word_embeddings=False, factor=8.0),
}
# requests, prompt lengths, new tokens, token budget of a step, seed of the weights
WORKLOADS = {
    "3b": dict(requests=64, prompt=(128, 2048), gen=(256, 256), max_prefill=512, seed=5, arrive_over=0.0),
    "1b": dict(requests=256, prompt=(16, 1024), gen=(32, 512), max_prefill=1024, seed=6, arrive_over=1.0),
    "8b": dict(requests=32, prompt=(128, 2048), gen=(128, 128), max_prefill=2048, seed=4, arrive_over=0.0),
}


def peaks() -> dict:
    """Measured peaks of this machine's GPU (MEASURED_PEAKS.json at the repository's root), else
    the figures of an earlier measurement on the same kind of GPU."""
    path = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if path.is_file():
        p = json.loads(path.read_text())
        return dict(hbm_gbs=p["hbm_gbs"], tflops=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1400.0, source="fallback")


def arrival_times(n: int, span: float, seed: int):
    """Seeded arrival times of ``n`` requests: exponential gaps scaled so that the last request
    arrives ``span`` seconds after the first."""
    rng = random.Random(2000 + seed)
    t, times = 0.0, []
    for _ in range(n):
        times.append(t)
        t += rng.expovariate(1.0)
    scale = span / times[-1] if n > 1 and times[-1] > 0 else 0.0
    return [x * scale for x in times]


def roofline_of(log, cfg: dict, weight_bytes: int, kv_bytes_per_token: int, max_prefill: int, pk: dict) -> dict:
    """What the steps of ``log`` (entries of ``Fastgen.step_log``) achieved."""
    d, f, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hq, hkv, hd, layers = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["num_hidden_layers"]
    matmul = layers * (d * (hq + 2 * hkv) * hd + hq * hd * d + 3 * d * f)
    decode = [s for s in log if s["prompt_tokens"] == 0 and s["decode_tokens"] > 0]
    heavy = [s for s in log if s["prompt_tokens"] >= max_prefill // 2]
    mixed = [s for s in log if s["prompt_tokens"] > 0 and s["decode_tokens"] > 0]
    out = {"steps_decode_only": len(decode), "steps_prompt_heavy": len(heavy), "steps_mixed": len(mixed),
           "mixed_share": round(len(mixed) / max(1, len(log)), 3), "peaks": pk["source"]}
    if decode:
        seconds = sum(s["t_end"] - s["t_start"] for s in decode)
        read = sum(weight_bytes + s["kv_tokens"] * kv_bytes_per_token for s in decode)
        out["decode_hbm_gbs"] = round(read / seconds / 1e9, 1)
        out["decode_hbm_frac"] = round(read / seconds / 1e9 / pk["hbm_gbs"], 4)
        out["decode_mean_batch"] = round(sum(s["decode_tokens"] for s in decode) / len(decode), 1)
    if heavy:
        seconds = sum(s["t_end"] - s["t_start"] for s in heavy)
        flops = sum(2 * matmul * (s["prompt_tokens"] + s["decode_tokens"]) + 4 * hd * hq * layers * s["key_pairs"]
                    + 2 * d * v * max(1, s["decode_tokens"]) for s in heavy)
        out["prompt_tflops"] = round(flops / seconds / 1e12, 1)
        out["prompt_tensor_frac"] = round(flops / seconds / 1e12 / pk["tflops"], 4)
    return out


def config_of(shape: str, layers: int = 0) -> dict:
    s = SHAPES[shape]
    return dict(
        architectures=["LlamaForCausalLM"], hidden_size=s["hidden_size"], intermediate_size=s["intermediate_size"],
        num_hidden_layers=layers or s["num_hidden_layers"], num_attention_heads=s["num_attention_heads"],
        num_key_value_heads=s["num_key_value_heads"], head_dim=s["head_dim"], rms_norm_eps=1e-5,
        vocab_size=128256, tie_word_embeddings=s["tie_word_embeddings"], rope_theta=500000.0,
        rope_scaling=dict(factor=s["factor"], low_freq_factor=1.0, high_freq_factor=4.0,
                          original_max_position_embeddings=8192, rope_type="llama3"),
        max_position_embeddings=131072,
    )


def make_requests(shape: str, n: int = 0, seed: int = 0):
    """[(prompt tokens, new tokens)] of the shape's workload, from a seeded host generator."""
    w = WORKLOADS[shape]
    rng = random.Random(1000 + seed)
    out = []
    for _ in range(n or w["requests"]):
        p = rng.randint(*w["prompt"])
        g = rng.randint(*w["gen"])
        out.append(([rng.randrange(128256) for _ in range(p)], g))
    return out


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--shape", choices=sorted(SHAPES), default="3b")
    ap.add_argument("--requests", type=int, default=0, help="number of requests (0: the workload's own)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (0: all)")
    ap.add_argument("--max-batch", type=int, default=0, help="requests decoding at once (0: all of them)")
    ap.add_argument("--max-prefill", type=int, default=0, help="tokens a step (0: the workload's own)")
    ap.add_argument("--sync-freq", type=int, default=10)
    ap.add_argument("--page", type=int, default=64)
    ap.add_argument("--graphs", type=int, default=32, help="most decode graphs (batch buckets)")
    ap.add_argument("--arrive-over", type=float, default=None,
                    help="seconds over which the requests arrive (0: all at once; default: the workload's own)")
    args = ap.parse_args()

    import torch

    from fastgen_b200.config import model_args_from_config
    from fastgen_b200.engine import Fastgen, GenArgs, Model, Packet

    w = WORKLOADS[args.shape]
    cfg = config_of(args.shape, args.layers)
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    model = Model.random(model_args_from_config(cfg), torch.bfloat16, dev, seed=w["seed"])
    reqs = make_requests(args.shape, args.requests)
    max_batch = args.max_batch or len(reqs)
    longest = sorted((len(p) + g for p, g in reqs), reverse=True)[:max_batch]
    max_seq = sum(-(-(n + 1) // args.page) * args.page for n in longest) + 2 * args.page
    gen_args = GenArgs(use_sampling=False, max_batch=max_batch, max_seq=max_seq, cache_block=args.page,
                       max_prefill=args.max_prefill or w["max_prefill"], num_cuda_graphs=min(max_batch, args.graphs),
                       sync_freq=args.sync_freq)
    fg = Fastgen(gen_args, model, stop_tokens=[])

    span = w["arrive_over"] if args.arrive_over is None else args.arrive_over
    arrivals = arrival_times(len(reqs), span, w["seed"]) if span > 0 else None

    def run(items):
        q = queue.Queue()
        packets = [Packet(thread_id=i, tokens=p, max_gen=g) for i, (p, g) in enumerate(items)]
        producer = None
        if arrivals is None:
            for pkt in packets:
                q.put(pkt)
            q.put(None)
        else:
            def produce(t_begin):
                for pkt, at in zip(packets, arrivals):
                    delay = t_begin + at - time.perf_counter()
                    if delay > 0:
                        time.sleep(delay)
                    q.put(pkt)
                q.put(None)
            producer = threading.Thread(target=produce, args=(time.perf_counter(),), daemon=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        if producer is not None:
            producer.start()
        n_out, errors = 0, 0
        for pkt in fg.generate(q):
            n_out += len(pkt.tokens)
            errors += pkt.error is not None
        torch.cuda.synchronize()
        return time.perf_counter() - t0, n_out, errors

    # warm-up: the same workload once (libraries load, the decode graphs of every batch and
        # context bucket it visits are captured); a server pays this once, not per request
    first_seconds, _, _ = run(reqs)
    steps0, pre0, log0 = fg.steps, fg.scheduler.n_preemptions, len(fg.step_log)
    seconds, n_out, errors = run(reqs)
    roofline = roofline_of(fg.step_log[log0:], cfg, model.weight_bytes(), model.cache_bytes_per_token(2),
                           gen_args.max_prefill, peaks())
    n_prompt = sum(len(p) for p, _ in reqs)
    line = {
        "impl": "ours", "workload": f"llama-{args.shape} shape, continuous batching", "requests": len(reqs),
        "layers": cfg["num_hidden_layers"], "prompt_tokens": n_prompt, "generated_tokens": n_out,
        "seconds": round(seconds, 3), "first_run_seconds": round(first_seconds, 3), "generated_tok_s": round(n_out / seconds, 1),
        "total_tok_s": round((n_out + n_prompt) / seconds, 1), "steps": fg.steps - steps0,
        "preemptions": fg.scheduler.n_preemptions - pre0, "errors": errors, "max_batch": max_batch,
        "max_prefill": gen_args.max_prefill, "sync_freq": gen_args.sync_freq, "page": args.page,
        "arrive_over_s": span, "roofline": roofline,
        "timing": "wall clock around generate(), host tokens in and out",
    }
    fg.destroy()
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
