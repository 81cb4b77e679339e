"""The reference arm of bench.py: the unmodified reference, installed under
``baseline/_ref``, driven through its own public API
(``Fastgen.build(loader, GenArgs(...))`` and ``fg.generate(queue)``).

Nothing of fastgen_b200 is on this path.  The reference has no random-weights
mode and wants tokenizer files, so the arm brings a loader of its own -- a
subclass of the reference's ``BaseLoader``, which is the extension point the
reference provides -- that describes the Llama-3.1-8B shape, fills the
parameters with N(0, 0.02) and hands out a tokenizer stub without stop tokens.

Decode throughput is what ``generate`` adds per step once the prompts are in:
the same prompts are generated twice, for ``warmup`` and for ``warmup + steps``
new tokens, and the difference of the wall-clock times is divided into the
difference of the generated tokens.  (The reference's generator has no hook to
time its decode phase alone, and its time per request includes host work by
design, so for this arm ``value`` and ``e2e`` are the same number.)
"""

from __future__ import annotations

import os
import queue
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent


def _unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}


def run(args, cfg: dict) -> dict:
    ref = HERE / "_ref"
    if not (ref / "fastgen").is_dir():
        return _unavailable("the reference is not installed under baseline/_ref")
    sys.path.insert(0, str(ref))
    try:
        import torch
        from fastgen.generate import Fastgen, GenArgs, Packet
        from fastgen.model import ModelArgs, RopeArgs
        from fastgen.utils.loading import BaseLoader
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"the reference does not import here: {e!r}")

    class StubTokenizer:
        stop_tokens: list = []
        vocab_size = cfg["vocab_size"]

    class RandomLoader(BaseLoader):
        def load_model_args(self):
            sc = cfg["rope_scaling"]
            return ModelArgs(
                dim=cfg["hidden_size"], ffn_dim=cfg["intermediate_size"], n_layers=args.layers or cfg["num_hidden_layers"],
                n_heads=cfg["num_attention_heads"], n_kv_heads=cfg["num_key_value_heads"], qkv_bias=False,
                norm_eps=cfg["rms_norm_eps"], vocab_size=cfg["vocab_size"], vocab_parallel=False, tie_embeddings=False,
                rope=RopeArgs(theta=cfg["rope_theta"], use_scaled_rope=True,
                              old_context_len=sc["original_max_position_embeddings"], scale_factor=sc["factor"],
                              low_freq_factor=sc["low_freq_factor"], high_freq_factor=sc["high_freq_factor"]),
            )

        def load_tokenizer(self):
            return StubTokenizer()

        def load(self, model, show_progress: bool = True) -> None:
            gen = torch.Generator(device="cuda").manual_seed(4)
            with torch.no_grad():
                for name, p in model.named_parameters():
                    if name.endswith("norm.weight"):
                        p.fill_(1.0)
                    else:
                        p.normal_(0.0, 0.02, generator=gen)

    try:
        torch.manual_seed(777)
        device = torch.device("cuda:0")
        torch.cuda.set_device(device)
        torch.set_default_device(device)  # as the reference's own tools do (fastgen/tools/chat.py:47-48)
        k, w, batch, ctx = args.steps, args.warmup, args.batch, args.context
        prompt_len = max(1, ctx - k - w)
        block = 256  # the reference's default cache_block
        per_lane = -(-(ctx + block) // block) * block
        gen_args = GenArgs(use_sampling=False, max_batch=batch, max_seq=max(batch * per_lane, 2048 + 2 * block),
                           max_gen=k + w, host_cache_gb=0)
        fg = Fastgen.build(RandomLoader(), gen_args, tp_mesh=None, device=device, profile_sig=None)
        g = torch.Generator(device="cpu").manual_seed(4)

        def prompts(n, length):
            return [torch.randint(0, cfg["vocab_size"], (length,), generator=g, device="cpu").tolist()
                    for _ in range(n)]

        def generate(ps, max_gen):
            q = queue.Queue()
            for i, p in enumerate(ps):
                q.put(Packet(thread_id=i, tokens=p, max_gen=max_gen))
            q.put(None)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            n = sum(len(pkt.tokens) for pkt in fg.generate(q))
            torch.cuda.synchronize()
            return time.perf_counter() - t0, n

        ps = prompts(batch, prompt_len)
        generate(ps, 2)  # warm-up: Triton compiles, graphs are already captured by build()
        t_short, n_short = generate(ps, w)
        t_long, n_long = generate(ps, w + k)
        decode_tok_s = (n_long - n_short) / (t_long - t_short)
        ms_per_step = (t_long - t_short) / k * 1e3
        one = prompts(1, 2048)
        for _ in range(3):
            generate(one, 1)
        t_pre = min(generate(one, 1)[0] for _ in range(5))
        fg.destroy()
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"the reference failed on this box: {e!r}")
    return {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (8B, bf16)",
        "value": round(decode_tok_s, 1), "unit": "tokens/s", "n_gpus": 1, "steps": k, "warmup": w,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights seed 4, uniform random token ids)",
        "impl": "reference",
        "config": {"model": "Llama-3.1-8B shape", "global_batch": batch, "seq_len": ctx, "parallelism": "single GPU",
                   "layers": args.layers or cfg["num_hidden_layers"], "layers_full": cfg["num_hidden_layers"],
                   "page": block, "prefill_tokens": 2048,
                   "timing": "wall clock around generate(); decode = difference of two runs"},
        "prefill": {"value": round(2048 / t_pre, 1), "tokens": 2048, "ms": round(t_pre * 1e3, 3)},
        "e2e": {"value": round(decode_tok_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": None,
                "d2h_bytes_per_step": None},
    }
