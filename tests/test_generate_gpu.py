"""Generation through the Python entry point and the command line."""

import queue
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers as H
import plain_llama as pl

pytestmark = pytest.mark.gpu


def _generate(model_dir, prompts, dtype, **kw):
    from fastgen_b200.engine import Fastgen, GenArgs, HfLoader, Packet

    args = GenArgs(**kw)
    fg = Fastgen.build(HfLoader(model_dir), args, tp_mesh=None, device=torch.device("cuda:0"), dtype=dtype)
    q = queue.Queue()
    for i, p in enumerate(prompts):
        q.put(Packet(thread_id=i, tokens=p))
    q.put(None)
    out = {pkt.thread_id: pkt for pkt in fg.generate(q)}
    stats = dict(preemptions=fg.scheduler.n_preemptions, steps=fg.steps)
    fg.engine.cache.check()
    assert fg.engine.cache.n_live == 0
    fg.destroy()
    return out, stats


def test_greedy_generation_equals_plain(tmp_path):
    """tiny-A workload: prompts 7, 13, 1, 30; 16 greedy tokens; pages of 8 (float32)."""
    model_dir = H.make_model_dir(tmp_path, "tiny_a")
    prompts = [H.random_tokens(256, n, 1 + i) for i, n in enumerate([7, 13, 1, 30])]
    out, _ = _generate(model_dir, prompts, torch.float32, use_sampling=False, max_gen=16,
                       cache_block=8, max_seq=256, max_batch=4, max_prefill=16)
    model = pl.read_model(model_dir)
    for i, p in enumerate(prompts):
        assert out[i].tokens == pl.greedy(model, p, 16), f"prompt {i}"


def test_greedy_with_preemption_equals_plain(tmp_path):
    """So few pages that requests are preempted and recomputed; tokens do not change."""
    model_dir = H.make_model_dir(tmp_path, "tiny_b")
    prompts = [H.random_tokens(320, n, 10 + i) for i, n in enumerate([9, 40, 24, 17])]
    out, stats = _generate(model_dir, prompts, torch.float32, use_sampling=False, max_gen=12,
                           cache_block=16, max_seq=96, max_batch=4, max_prefill=16)
    assert stats["preemptions"] >= 1
    model = pl.read_model(model_dir)
    for i, p in enumerate(prompts):
        assert out[i].tokens == pl.greedy(model, p, 12), f"prompt {i}"


def test_bf16_greedy_follows_plain_where_the_margin_is_clear(tmp_path):
    model_dir = H.make_model_dir(tmp_path, "tiny_b", std=0.08)
    prompts = [H.random_tokens(320, n, 20 + i) for i, n in enumerate([5, 33])]
    out, _ = _generate(model_dir, prompts, torch.bfloat16, use_sampling=False, max_gen=8,
                       cache_block=16, max_seq=256, max_batch=2)
    model = pl.read_model(model_dir)
    for i, p in enumerate(prompts):
        seq = list(p)
        for tok in out[i].tokens:
            logits = pl.forward(model, seq)[-1].numpy()
            # the engine's token is the plain argmax, or within bfloat16 error of it
            assert logits[tok] >= logits.max() - H.BF16_MAX * np.abs(logits).max()
            seq.append(tok)


def test_sampling_is_seeded_and_independent_of_batching(tmp_path):
    """tiny-B workload: temperature 0.8, seeded; prompts prefilled in portions of 16
    beside decoding requests give the same tokens as each request alone."""
    model_dir = H.make_model_dir(tmp_path, "tiny_b")
    prompts = [H.random_tokens(320, n, 3 + i) for i, n in enumerate([1, 9, 40, 64, 100])]
    kw = dict(use_sampling=True, temperature=0.8, top_p=0.9, max_gen=24, cache_block=16,
              max_seq=512, seed=5, logprobs=True)
    together, _ = _generate(model_dir, prompts, torch.float32, max_batch=4, max_prefill=16, **kw)
    again, _ = _generate(model_dir, prompts, torch.float32, max_batch=4, max_prefill=16, **kw)
    other, _ = _generate(model_dir, prompts, torch.float32, max_batch=4, max_prefill=16, **dict(kw, seed=6))
    for i in range(len(prompts)):
        assert together[i].tokens == again[i].tokens
        assert len(together[i].tokens) == 24 and len(together[i].logprobs) == 24
    assert any(together[i].tokens != other[i].tokens for i in range(len(prompts)))
    # alone: same request keys are needed for the same draws, so run them in the same order, one lane
    alone, _ = _generate(model_dir, prompts, torch.float32, max_batch=1, max_prefill=512, **kw)
    same = sum(together[i].tokens == alone[i].tokens for i in range(len(prompts)))
    assert same == len(prompts)
    # logprobs are those of the plain implementation
    model = pl.read_model(model_dir)
    seq = prompts[1] + together[1].tokens
    logits = pl.forward(model, seq[:-1])
    lp = torch.log_softmax(logits.double(), -1)
    for k, tok in enumerate(together[1].tokens):
        assert abs(float(lp[len(prompts[1]) - 1 + k, tok]) - together[1].logprobs[k]) < 1e-3


def test_sync_freq_does_not_change_tokens(tmp_path):
    """Runs of 1, 3, 10 or 64 decode steps between two reads of the sampled tokens give the
    same tokens: greedy in bfloat16 at head size 64 (keys beyond one split), and sampled in
    float32, with a stop token that falls inside a run."""
    model_dir = H.make_model_dir(tmp_path, "tiny_d")
    prompts = [H.random_tokens(300, n, 40 + i) for i, n in enumerate([3, 140, 70])]
    ref = None
    for freq in (1, 3, 10, 64):
        out, _ = _generate(model_dir, prompts, torch.bfloat16, use_sampling=False, max_gen=40, cache_block=64,
                           max_seq=1024, max_batch=4, sync_freq=freq)
        toks = [out[i].tokens for i in range(len(prompts))]
        assert all(len(t) == 40 for t in toks)
        ref = ref or toks
        assert toks == ref, f"sync_freq {freq}"

    from fastgen_b200.engine import Fastgen, GenArgs, HfLoader, Packet
    model_dir = H.make_model_dir(tmp_path, "tiny_b")
    prompts = [H.random_tokens(320, n, 3 + i) for i, n in enumerate([9, 40, 1])]
    ref = None
    for freq in (1, 4, 10):
        fg = Fastgen.build(HfLoader(model_dir), GenArgs(use_sampling=True, temperature=0.8, top_p=0.9, max_gen=30,
                                                        cache_block=16, max_seq=512, seed=5, max_batch=4,
                                                        sync_freq=freq), device="cuda:0", dtype=torch.float32)
        if ref is not None:
            fg.scheduler.stop_tokens = {ref[0][13]}  # falls inside a run of the first request
        q = queue.Queue()
        for i, p in enumerate(prompts):
            q.put(Packet(thread_id=i, tokens=p))
        q.put(None)
        out = {pkt.thread_id: pkt.tokens for pkt in fg.generate(q)}
        fg.destroy()
        if ref is None:
            ref = out
            continue
        stop = ref[0][13]
        for i in range(len(prompts)):
            want = ref[i][: ref[i].index(stop) + 1] if stop in ref[i] else ref[i]
            assert out[i] == want, f"sync_freq {freq}, request {i}"


@pytest.mark.parametrize("sampling", [False, True])
def test_many_requests_under_preemption_keep_their_tokens(tmp_path, sampling):
    """Forty requests of random lengths through a cache that holds a few of them: requests are
    preempted and recomputed again and again (decode runs of 10 steps included), and in
    float32 every request still gets the tokens it gets with room for all."""
    import random
    from fastgen_b200.engine import Fastgen, GenArgs, HfLoader, Packet

    model_dir = H.make_model_dir(tmp_path, "tiny_d")
    rng = random.Random(5)
    prompts = [H.random_tokens(300, rng.randint(1, 200), 100 + i) for i in range(40)]
    gens = [rng.randint(1, 120) for _ in prompts]

    def run(max_seq):
        fg = Fastgen.build(HfLoader(model_dir), GenArgs(use_sampling=sampling, temperature=0.9, top_p=0.95,
                                                        cache_block=64, max_seq=max_seq, max_batch=16, max_prefill=128,
                                                        seed=3), device="cuda:0", dtype=torch.float32)
        q = queue.Queue()
        for i, (p, g) in enumerate(zip(prompts, gens)):
            q.put(Packet(thread_id=i, tokens=p, max_gen=g))
        q.put(None)
        out = {p.thread_id: p.tokens for p in fg.generate(q)}
        n = fg.scheduler.n_preemptions
        fg.engine.cache.check()
        assert fg.engine.cache.n_live == 0
        fg.destroy()
        return out, n

    roomy, n_roomy = run(16 * 384)
    tight, n_tight = run(6 * 64 + 320)
    assert n_roomy == 0 and n_tight >= 5
    assert all(len(roomy[i]) == gens[i] for i in roomy)
    assert tight == roomy


def test_profile_trace_on_request(tmp_path, monkeypatch):
    """request_profile() traces the next FG_PROFILE_ITERS iterations into FG_PROFILE_DIR."""
    import gzip
    from fastgen_b200.engine import Fastgen, GenArgs, HfLoader, Packet

    monkeypatch.setenv("FG_PROFILE_ITERS", "3")
    monkeypatch.setenv("FG_PROFILE_DIR", str(tmp_path))
    model_dir = H.make_model_dir(tmp_path, "tiny_a")
    fg = Fastgen.build(HfLoader(model_dir), GenArgs(use_sampling=False, max_gen=12, cache_block=8, max_seq=128,
                                                    max_batch=2, sync_freq=1), device="cuda:0", dtype=torch.float32)
    fg.request_profile()
    q = queue.Queue()
    q.put(Packet(thread_id=0, tokens=H.random_tokens(256, 9, 1)))
    q.put(None)
    out = list(fg.generate(q))
    assert len(out) == 1 and len(out[0].tokens) == 12
    assert fg.profile_state == "inactive" and fg.last_profile is not None
    with gzip.open(fg.last_profile, "rt") as f:
        head = f.read(4096)
    assert "traceEvents" in head
    fg.destroy()


def test_stop_token_and_errors(tmp_path):
    model_dir = H.make_model_dir(tmp_path, "tiny_a")
    model = pl.read_model(model_dir)
    prompt = H.random_tokens(256, 7, 1)
    ref = pl.greedy(model, prompt, 16)
    from fastgen_b200.engine import Fastgen, GenArgs, HfLoader, Packet

    fg = Fastgen.build(HfLoader(model_dir), GenArgs(use_sampling=False, max_gen=16, cache_block=8, max_seq=64,
                                                    max_batch=2), device="cuda:0", dtype=torch.float32)
    fg.scheduler.stop_tokens = {ref[3]}
    q = queue.Queue()
    q.put(Packet(thread_id="stop", tokens=prompt))
    q.put(Packet(thread_id="long", tokens=H.random_tokens(256, 80, 2)))
    q.put(Packet(thread_id="capped", tokens=prompt, max_gen=2))
    q.put(None)
    out = {p.thread_id: p for p in fg.generate(q)}
    first = ref.index(ref[3])
    assert out["stop"].tokens == ref[: first + 1]
    assert out["long"].error and out["long"].tokens == []
    assert len(out["capped"].tokens) <= 2
    fg.destroy()


def test_fgchat_token_id_mode(tmp_path):
    model_dir = H.make_model_dir(tmp_path, "tiny_a")
    root = Path(__file__).resolve().parent.parent
    proc = subprocess.run(
        [sys.executable, str(root / "bin" / "fgchat"), str(model_dir), "--temperature", "0.0",
         "--max-tokens", "6", "--dtype", "fp32", "--page-size", "8", "--max-seq", "128"],
        input="5 17 3 200\n/q\n", text=True, capture_output=True, timeout=600,
    )
    assert proc.returncode == 0, proc.stderr[-2000:]
    ref = pl.greedy(pl.read_model(model_dir), [5, 17, 3, 200], 6)
    assert " ".join(map(str, ref)) in proc.stdout
    assert "--- [6 tokens," in proc.stdout


def test_fgchat_token_id_mode_keeps_the_conversation(tmp_path):
    """The second round's prompt is the first prompt, the first answer and the new line; ``/r 2``
    goes back to the state before the second exchange."""
    import re
    model_dir = H.make_model_dir(tmp_path, "tiny_b", std=0.08)  # weights under which the history matters
    root = Path(__file__).resolve().parent.parent
    proc = subprocess.run(
        [sys.executable, str(root / "bin" / "fgchat"), str(model_dir), "--temperature", "0.0",
         "--max-tokens", "5", "--dtype", "fp32", "--page-size", "8", "--max-seq", "128"],
        input="5 17 3 200\n9 9 41\n/r 2\n77 1\n/q\n", text=True, capture_output=True, timeout=600,
    )
    assert proc.returncode == 0, proc.stderr[-2000:]
    model = pl.read_model(model_dir)
    first = pl.greedy(model, [5, 17, 3, 200], 5)
    second = pl.greedy(model, [5, 17, 3, 200] + first + [9, 9, 41], 5)
    again = pl.greedy(model, [5, 17, 3, 200] + first + [77, 1], 5)
    assert second != pl.greedy(model, [9, 9, 41], 5) and again != pl.greedy(model, [77, 1], 5)
    lines = [re.sub(r"^(\d+> )+", "", l) for l in proc.stdout.splitlines()]  # the prompts share the answers' lines
    answers = [l for l in lines if l and all(c.isdigit() or c == " " for c in l)]
    assert answers == [" ".join(map(str, t)) for t in (first, second, again)], proc.stdout


@pytest.mark.parametrize("when", ["first step", "a run of decode steps"])
def test_a_kernel_fault_surfaces_through_generate(tmp_path, when):
    """A block-table entry that is wrong on the device (here: set to -1 behind the host's back)
    makes the kernels record the fault and skip the access; the generator reads the status word
    with the sampled tokens, ends the step's requests with an error and goes on clean."""
    from fastgen_b200.engine import Fastgen, GenArgs, HfLoader, Packet

    model_dir = H.make_model_dir(tmp_path, "tiny_d")
    prompts = [H.random_tokens(300, n, 60 + i) for i, n in enumerate([70, 5, 33])]
    fg = Fastgen.build(HfLoader(model_dir), GenArgs(use_sampling=False, max_gen=12, cache_block=64, max_seq=1024,
                                                    max_batch=4, sync_freq=10),
                       tp_mesh=None, device=torch.device("cuda:0"), dtype=torch.bfloat16)

    def run():
        q = queue.Queue()
        for i, p in enumerate(prompts):
            q.put(Packet(thread_id=i, tokens=p))
        q.put(None)
        return {pkt.thread_id: pkt for pkt in fg.generate(q)}

    clean = run()
    assert all(p.error is None and len(p.tokens) == 12 for p in clean.values())
    cache = fg.engine.cache
    flush, broken = cache.flush_tables, {"on": True, "calls": 0}

    def flush_then_break():
        # the tables are flushed once before the step that takes the prompts, then once
        # before the run of decode steps
        flush()
        broken["calls"] += 1
        if broken["on"] and broken["calls"] >= (1 if when == "first step" else 2):
            for req in cache._requests.values():
                cache.groups[0].device_table[req.slot, 0] = -1

    cache.flush_tables = flush_then_break
    out = run()
    assert len(out) == 3
    for pkt in out.values():
        assert pkt.error is not None and "block-table entry" in pkt.error, pkt
    assert cache.n_live == 0 and int(fg.ops.status.item()) == 0
    cache.check()
    # the generator is usable afterwards and gives what it gave before
    broken["on"] = False
    again = run()
    assert {i: p.tokens for i, p in again.items()} == {i: p.tokens for i, p in clean.items()}
    fg.destroy()


def test_cache_size_from_the_memory_budget(tmp_path):
    """``max_seq < 0`` (the default of ``GenArgs``): the cache gets what ``gpu_gb`` leaves after
    the weights and ``prefill_gb`` (fastgen/utils/tune.py:31-84, fastgen/generate.py:206-236)."""
    from fastgen_b200.engine import Fastgen, GenArgs, HfLoader, Packet

    model_dir = H.make_model_dir(tmp_path, "tiny_b")
    prompts = [H.random_tokens(320, n, 80 + i) for i, n in enumerate([9, 40])]
    args = GenArgs(use_sampling=False, max_gen=8, cache_block=16, max_batch=4, gpu_gb=0.11, prefill_gb=0.1)
    assert args.max_seq < 0 and args.num_cuda_graphs == 16
    fg = Fastgen.build(HfLoader(model_dir), args, tp_mesh=None, device=torch.device("cuda:0"), dtype=torch.float32)
    per_token = 2 * 3 * 3 * 32 * 4  # keys and values, 3 layers, 3 heads of 32, float32
    expect = (int(0.11e9) - fg.model.weight_bytes() - int(0.1e9)) // per_token
    expect = -(-expect // 16) * 16
    assert fg.max_seq == expect and 1000 < expect < 3000
    assert fg.engine.cache.groups[0].pool.n_pages == expect // 16
    q = queue.Queue()
    for i, p in enumerate(prompts):
        q.put(Packet(thread_id=i, tokens=p))
    q.put(None)
    out = {pkt.thread_id: pkt.tokens for pkt in fg.generate(q)}
    model = pl.read_model(model_dir)
    for i, p in enumerate(prompts):
        assert out[i] == pl.greedy(model, p, 8)
    fg.destroy()
    with pytest.raises(RuntimeError, match="Not enough memory"):
        Fastgen.build(HfLoader(model_dir), GenArgs(cache_block=16, gpu_gb=0.1, prefill_gb=0.1), tp_mesh=None,
                      device=torch.device("cuda:0"), dtype=torch.float32)


def test_default_gen_args_pad_their_graphs(tmp_path):
    """``GenArgs()`` as shipped: 256 lanes and 16 graph buckets (1, 18, 35, ...), so a handful of
    requests decode in a graph of 18 lanes.  Greedy tokens equal the plain implementation's."""
    from fastgen_b200.engine import Fastgen, GenArgs, HfLoader, Packet

    model_dir = H.make_model_dir(tmp_path, "tiny_b")
    prompts = [H.random_tokens(320, n, 90 + i) for i, n in enumerate([9, 40, 3, 77, 21])]
    args = GenArgs(use_sampling=False, max_gen=10, cache_block=16, gpu_gb=0.12, prefill_gb=0.1)
    fg = Fastgen.build(HfLoader(model_dir), args, tp_mesh=None, device=torch.device("cuda:0"), dtype=torch.float32)
    assert fg.max_batch == 256 and sorted(fg.engine.graphs.buckets)[:3] == [1, 18, 35]
    q = queue.Queue()
    for i, p in enumerate(prompts):
        q.put(Packet(thread_id=i, tokens=p))
    q.put(None)
    out = {pkt.thread_id: pkt.tokens for pkt in fg.generate(q)}
    assert fg.engine.graphs.padded_replays >= 5
    model = pl.read_model(model_dir)
    for i, p in enumerate(prompts):
        assert out[i] == pl.greedy(model, p, 10)
    fg.destroy()


def test_fgchat_text_mode_with_a_tokenizer(tmp_path):
    """A model folder with tokenizer files: the dialog goes through the chat template, the answer
    comes back as text, and the stop token (the tokenizer's eos) ends it."""
    import json
    import re
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import WhitespaceSplit

    model_dir = H.make_model_dir(tmp_path, "tiny_a")
    words = ["<s>", "</s>", "<unk>", "user", "assistant", ":", "hello", "world", "how", "are", "you"] + \
            [f"w{i}" for i in range(11, 256)]
    tk = Tokenizer(WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tk.pre_tokenizer = WhitespaceSplit()
    tk.save(str(model_dir / "tokenizer.json"))
    template = ("{{ bos_token }} {% for m in messages %}{{ m['role'] }} : {{ m['content'] }} {% endfor %}"
                "{% if add_generation_prompt %}assistant :{% endif %}")
    (model_dir / "tokenizer_config.json").write_text(
        json.dumps(dict(bos_token="<s>", eos_token="</s>", chat_template=template)))
    root = Path(__file__).resolve().parent.parent
    proc = subprocess.run(
        [sys.executable, str(root / "bin" / "fgchat"), str(model_dir), "--temperature", "0.0",
         "--max-tokens", "6", "--dtype", "fp32", "--page-size", "8", "--max-seq", "128"],
        input="hello world\nhow are you\n/q\n", text=True, capture_output=True, timeout=600,
    )
    assert proc.returncode == 0, proc.stderr[-2000:]
    model = pl.read_model(model_dir)
    ids = lambda text: [words.index(w) for w in text.split()]
    first_prompt = ids("<s> user : hello world assistant :")
    first = pl.greedy(model, first_prompt, 6)
    if 1 in first:  # the eos token ends an answer and is not shown
        first = first[: first.index(1) + 1]
    shown = [t for t in first if t != 1] if first and first[-1] == 1 else first
    lines = [re.sub(r"^(\d+> )+", "", l) for l in proc.stdout.splitlines()]
    assert " ".join(words[t] for t in shown) in lines, proc.stdout
    assert f"--- [{len(first)} tokens," in proc.stdout
    second_prompt = ids("<s> user : hello world assistant : " + " ".join(words[t] for t in shown) +
                        " user : how are you assistant :")
    second = pl.greedy(model, second_prompt, 6)
    if 1 in second:
        second = second[: second.index(1) + 1]
    shown2 = [t for t in second if t != 1] if second and second[-1] == 1 else second
    assert " ".join(words[t] for t in shown2) in lines, proc.stdout
