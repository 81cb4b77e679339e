"""The continuous-batching workloads of ``fastgen_b200.tools.serve_bench`` through the
unmodified reference (installed under ``baseline/_ref``), for a figure to set beside ours.

    python baseline/reference_serve.py --shape 3b

Nothing of fastgen_b200 runs here: only the workload table and the request generator are
read from its file (plain Python).  The reference gets random weights of the same shape
through a ``BaseLoader`` subclass, its own default page size (256) and its own scheduler
options; ``max_prefill`` is the workload's token budget.  One JSON line is printed, or
``{"impl": "reference", "unavailable": ...}``.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import queue
import sys
import threading
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent


def _workloads():
    spec = importlib.util.spec_from_file_location("serve_workloads", HERE.parent / "fastgen_b200" / "tools" / "serve_bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="3b")
    ap.add_argument("--requests", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--arrive-over", type=float, default=None,
                    help="seconds over which the requests arrive (0: all at once; default: the workload's own)")
    args = ap.parse_args()
    wl = _workloads()
    cfg = wl.config_of(args.shape, args.layers)
    w = wl.WORKLOADS[args.shape]
    ref = HERE / "_ref"
    if not (ref / "fastgen").is_dir():
        print(json.dumps({"impl": "reference", "unavailable": "the reference is not installed under baseline/_ref"}))
        return 0
    sys.path.insert(0, str(ref))
    try:
        import torch
        from fastgen.generate import Fastgen, GenArgs, Packet
        from fastgen.model import ModelArgs, RopeArgs
        from fastgen.utils.loading import BaseLoader

        class StubTokenizer:
            stop_tokens: list = []
            vocab_size = cfg["vocab_size"]

        class RandomLoader(BaseLoader):
            def load_model_args(self):
                sc = cfg["rope_scaling"]
                assert cfg["head_dim"] * cfg["num_attention_heads"] == cfg["hidden_size"]
                return ModelArgs(
                    dim=cfg["hidden_size"], ffn_dim=cfg["intermediate_size"], n_layers=cfg["num_hidden_layers"],
                    n_heads=cfg["num_attention_heads"], n_kv_heads=cfg["num_key_value_heads"], qkv_bias=False,
                    norm_eps=cfg["rms_norm_eps"], vocab_size=cfg["vocab_size"],
                    vocab_parallel=cfg["tie_word_embeddings"],  # as the reference's own loader sets it (utils/loading.py:71)
                    tie_embeddings=cfg["tie_word_embeddings"],
                    rope=RopeArgs(theta=cfg["rope_theta"], use_scaled_rope=True,
                                  old_context_len=sc["original_max_position_embeddings"], scale_factor=sc["factor"],
                                  low_freq_factor=sc["low_freq_factor"], high_freq_factor=sc["high_freq_factor"]),
                )

            def load_tokenizer(self):
                return StubTokenizer()

            def load(self, model, show_progress: bool = True) -> None:
                gen = torch.Generator(device="cuda").manual_seed(w["seed"])
                with torch.no_grad():
                    for name, p in model.named_parameters():
                        if name.endswith("norm.weight"):
                            p.fill_(1.0)
                        else:
                            p.normal_(0.0, 0.02, generator=gen)

        torch.manual_seed(777)
        device = torch.device("cuda:0")
        torch.cuda.set_device(device)
        torch.set_default_device(device)  # as the reference's own tools do (fastgen/tools/chat.py:47-48)
        reqs = wl.make_requests(args.shape, args.requests)
        block = 256
        max_batch = len(reqs)
        max_seq = sum(-(-(len(p) + g + 1) // block) * block for p, g in reqs) + 2 * block
        gen_args = GenArgs(use_sampling=False, max_batch=max_batch, max_seq=max_seq, host_cache_gb=0,
                           max_prefill=w["max_prefill"], min_prefill=min(2048, w["max_prefill"]))
        fg = Fastgen.build(RandomLoader(), gen_args, tp_mesh=None, device=device, profile_sig=None)

        span = w["arrive_over"] if args.arrive_over is None else args.arrive_over
        arrivals = wl.arrival_times(len(reqs), span, w["seed"]) if span > 0 else None

        def run(items):
            q = queue.Queue()
            packets = [Packet(thread_id=i, tokens=p, max_gen=g) for i, (p, g) in enumerate(items)]
            producer = None
            if arrivals is None:
                for pkt in packets:
                    q.put(pkt)
                q.put(None)
            else:  # the same seeded schedule as the other arm's
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
            n_out = sum(len(pkt.tokens) for pkt in fg.generate(q))
            torch.cuda.synchronize()
            return time.perf_counter() - t0, n_out

        first_seconds, _ = run(reqs)  # warm-up: the same workload once (Triton compiles)
        seconds, n_out = run(reqs)
        fg.destroy()
    except Exception as e:  # noqa: BLE001
        import traceback

        traceback.print_exc(file=sys.stderr)
        print(json.dumps({"impl": "reference", "unavailable": f"the reference failed on this box: {e!r}"[:300]}))
        return 0
    n_prompt = sum(len(p) for p, _ in reqs)
    print(json.dumps({
        "impl": "reference", "workload": f"llama-{args.shape} shape, continuous batching", "requests": len(reqs),
        "layers": cfg["num_hidden_layers"], "prompt_tokens": n_prompt, "generated_tokens": n_out,
        "seconds": round(seconds, 3), "first_run_seconds": round(first_seconds, 3), "generated_tok_s": round(n_out / seconds, 1),
        "total_tok_s": round((n_out + n_prompt) / seconds, 1), "max_batch": max_batch,
        "max_prefill": w["max_prefill"], "page": block, "arrive_over_s": span,
        "timing": "wall clock around generate(), host tokens in and out",
    }))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
