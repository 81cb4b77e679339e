"""``fgchat``-style command line (fastgen/tools/chat.py:87-220).

    python -m fastgen_b200.tools.chat MODEL_DIR [--temperature T] [--top-p P]
        [--max-tokens N] [--gpu-gb G] [--verbose]

Options of the reference keep their names and meanings: ``--temperature`` (0.7;
0.0 is greedy), ``--top-p`` (1.0 disables), ``--max-tokens``, ``--gpu-gb`` (20),
``--verbose``; ``--tensor-parallel`` is accepted with the value 1 only.  The
chat runs with ``max_batch=1`` as there.  Interactive commands: ``/r <N>`` reset
the conversation before round N, ``/m`` multi-line input ended by a single
``.``, ``/q`` quit.  After each answer ``--- [N tokens, X toks/s]`` is printed.

Added here: ``--dtype``, ``--page-size``, ``--seed`` and a token-id mode for
model folders without tokenizer files (random-weights folders): each input line
is a list of token ids and the answer is printed as token ids.
``--random-weights CONFIG.json`` first writes MODEL_DIR from that configuration.
"""

from __future__ import annotations

import argparse
import json
import logging
import queue
import time
from typing import List

import torch


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="fgchat")
    parser.add_argument("model", type=str, help="checkpoint directory (Hugging Face layout)")
    parser.add_argument("--tensor-parallel", type=int, default=1, help="must be 1: this engine uses one GPU")
    parser.add_argument("--verbose", action="store_true", help="enable logging")
    parser.add_argument("--temperature", type=float, default=0.7, help="sampling temperature (0.0 for greedy)")
    parser.add_argument("--top-p", type=float, default=1.0, help="top-p sampling (1.0 to disable)")
    parser.add_argument("--max-tokens", type=int, help="maximum number of tokens per answer")
    parser.add_argument("--gpu-gb", type=float, default=20, help="approximate amount of gpu memory to use")
    parser.add_argument("--dtype", choices=["bf16", "fp32"], default="bf16", help="compute dtype")
    parser.add_argument("--page-size", type=int, default=64, help="tokens per cache page")
    parser.add_argument("--seed", type=int, default=777, help="seed of the sampler")
    parser.add_argument("--random-weights", metavar="CONFIG", help="write MODEL from this config.json first")
    parser.add_argument("--max-seq", type=int, default=-1, help="cache size in tokens (default: from --gpu-gb)")
    return parser


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.tensor_parallel != 1:
        raise SystemExit("fgchat: this engine runs on one GPU; --tensor-parallel must be 1")
    logging.basicConfig(
        format="%(asctime)s %(levelname)-1.1s - %(message)s",
        level=logging.INFO if args.verbose else logging.WARNING,
    )
    from ..engine import Fastgen, GenArgs, HfLoader, Packet

    if args.random_weights:
        from ..weights import write_random_model

        with open(args.random_weights) as f:
            write_random_model(args.model, json.load(f), args.seed)

    loader = HfLoader(args.model)
    tokenizer = loader.load_tokenizer() if loader.has_tokenizer() else None
    gen_args = GenArgs(
        use_sampling=bool(args.temperature),
        temperature=args.temperature,
        top_p=args.top_p,
        max_batch=1,
        max_gen=args.max_tokens,
        gpu_gb=args.gpu_gb,
        cache_block=args.page_size,
        seed=args.seed,
        max_seq=args.max_seq,
    )
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    fg = Fastgen.build(loader, gen_args, tp_mesh=None, device=torch.device("cuda:0"), dtype=dtype)
    q: "queue.Queue" = queue.Queue()
    g = fg.generate(q)

    print("\u001b[32mReady to chat!\u001b[0m")
    print("  Available commands:")
    print("    /r <N> -- reset conversation before round N")
    print("    /m     -- input a multiline message, end your input")
    print("              with a single line containing '.'")
    print("    /q     -- quit")
    if tokenizer is None:
        print("  (no tokenizer files: type token ids, answers are token ids)")
    print("")
    print("---")

    dialog: List[dict] = []
    turns: List[List[int]] = []  # token-id mode: the conversation so far, a list per message
    while True:
        rnd = 1 + len(dialog) // 2
        try:
            msg = input(f"{rnd}> ").strip()
        except EOFError:
            print("^D")
            break
        if msg[:2] == "/q":
            break
        if msg[:2] == "/r":
            try:
                n = int(msg[2:].strip())
                dialog = dialog[: 2 * (n - 1)]
                turns = turns[: 2 * (n - 1)]
            except ValueError:
                print("invalid command")
            continue
        if msg[:2] == "/m":
            lines = []
            while True:
                line = input(f"{rnd}>> ")
                if line.strip() == ".":
                    break
                lines.append(line)
            msg = "\n".join(lines)
        if tokenizer is not None:
            dialog.append(dict(role="user", content=msg))
            tokens = tokenizer.encode_dialog(dialog)
        else:
            try:
                ids = [int(t) for t in msg.replace(",", " ").split()]
            except ValueError:
                print("invalid token ids")
                continue
            if not ids:
                continue
            dialog.append(dict(role="user", content=msg))
            turns.append(ids)
            # the conversation goes in whole, as a chat template would render it
            tokens = [t for turn in turns for t in turn]
        if not tokens:
            dialog.pop()
            continue
        t0 = time.monotonic()
        q.put(Packet(thread_id=0, tokens=tokens))
        pkt = next(g)
        tps = len(pkt.tokens) / max(time.monotonic() - t0, 1e-9)
        if pkt.error:
            print(f"error: {pkt.error}")
            dialog.pop()
            if tokenizer is None:
                turns.pop()
            continue
        ntoks = len(pkt.tokens)
        out = list(pkt.tokens)
        if out and out[-1] in fg.stop_tokens:
            out = out[:-1]
        text = tokenizer.decode(out) if tokenizer is not None else " ".join(map(str, out))
        dialog.append(dict(role="assistant", content=text))
        if tokenizer is None:
            turns.append(out)
        print(text)
        print(f"--- [{ntoks} tokens, {tps:.3f}toks/s]")

    q.put(None)
    for _ in g:
        pass
    fg.destroy()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
