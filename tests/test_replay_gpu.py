"""Replay through the engine, compared with the plain implementation."""

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
PAGES = {"tiny_a": 8, "tiny_b": 16, "tiny_c": 8, "tiny_d": 64, "tiny_e": 16}


def _requests(name, lengths, seed):
    vocab = H.CONFIGS[name][0]["vocab_size"]
    return {f"r{i}": H.random_tokens(vocab, n, seed + i) for i, n in enumerate(lengths)}


LENGTHS = {"tiny_a": [7, 13, 1, 30, 70], "tiny_b": [1, 9, 40, 64, 100], "tiny_c": [5, 33, 90, 64],
           "tiny_d": [3, 70, 200, 129, 330], "tiny_e": [5, 150, 260, 64]}


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", list(H.CONFIGS))
@pytest.mark.parametrize("plan", ["whole", "tail", "portions", "mixed"])
def test_replay(tmp_path, name, dtype, plan):
    model_dir = H.make_model_dir(tmp_path, name)
    reqs = _requests(name, LENGTHS[name], 100)
    page = PAGES[name]
    if plan == "whole":
        steps = H.plan_whole(reqs)
    elif plan == "tail":
        steps = H.plan_decode_tail(reqs)
    elif plan == "portions":
        steps = H.plan_portions(reqs)
    else:
        reqs = _requests(name, LENGTHS[name] + [48, 17, 80], 200)
        steps = H.plan_mixed(reqs, seed=5)
    # exactly as many pages as the trace needs at its fullest: pages are reused
    max_tokens = H.max_live_tokens(steps, page)
    outputs, engine = H.run_engine(model_dir, dtype, steps, page, max_tokens)
    got = H.collect(steps, outputs)
    H.compare(model_dir, reqs, got, dtype)
    assert engine.cache.n_live == 0
    assert all(f == g.pool.n_pages for f, g in zip(engine.cache.free_pages(), engine.cache.groups))


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["tiny_b", "tiny_c", "tiny_d", "tiny_e"])
@pytest.mark.parametrize("plan", ["portions", "mixed", "many"])
def test_replay_with_graphs_for_prompt_steps(tmp_path, name, dtype, plan):
    """The same replays with every step of up to 512 tokens replayed from a CUDA graph of its
    padded shape (tokens of slot -1 behind the step's own, tile lists padded with tiles of no
    request): prompt portions down to two tokens, portions beside decoded tokens, many
    requests.  What the generator does for steps up to its token budget."""
    model_dir = H.make_model_dir(tmp_path, name)
    page = PAGES[name]
    if plan == "portions":
        reqs = _requests(name, LENGTHS[name], 100)
        steps = H.plan_portions(reqs)
        kw = dict(max_requests=4)
    elif plan == "mixed":
        reqs = _requests(name, LENGTHS[name] + [48, 17, 80], 200)
        steps = H.plan_mixed(reqs, seed=5)
        kw = dict(max_requests=4)
    else:
        reqs = _requests(name, MANY.get(name, MANY["tiny_b"])[:12], 500)
        reqs = {k: v[: H.CONFIGS[name][0]["max_position_embeddings"] - 8] for k, v in reqs.items()}
        steps = H.plan_many(reqs, seed=9, max_live=10)
        kw = dict(max_requests=10, num_cuda_graphs=3)
    outputs, engine = H.run_engine(model_dir, dtype, steps, page, H.max_live_tokens(steps, page) + 2 * page,
                                   max_step_tokens=512, **kw)
    assert engine.step_graphs is not None and engine.step_graphs.replays >= 4
    got = H.collect(steps, outputs)
    H.compare(model_dir, reqs, got, dtype)
    assert engine.cache.n_live == 0


MANY = {"tiny_b": [30, 120, 75, 260, 41, 33, 180, 90, 64, 129, 200, 57, 310, 48, 150, 99],
        "tiny_d": [70, 300, 131, 420, 45, 260, 129, 64, 390, 200, 88, 333, 150, 257, 40, 512],
        "tiny_e": [50, 150, 260, 64, 129, 400, 33, 300, 210, 101, 99, 380, 45, 128, 256, 170]}


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", list(MANY))
def test_replay_many_live_requests_in_padded_graphs(tmp_path, name, dtype):
    """Up to 14 live requests and 3 graph buckets (1, 8, 14): most steps of single tokens
    replay a graph with more lanes than requests (lanes of slot -1), and with more than 8
    tokens a step bfloat16 takes the library product, the separate rotation and the separate
    gate.  Lengths cross several splits of 128 keys; the pool has three pages to spare, so
    pages are reused while others stay free."""
    model_dir = H.make_model_dir(tmp_path, name)
    reqs = _requests(name, MANY[name], 500)
    page = PAGES[name]
    steps = H.plan_many(reqs, seed=7, max_live=14)
    assert max(len(st["entries"]) for st in steps) == 14
    outputs, engine = H.run_engine(model_dir, dtype, steps, page, H.max_live_tokens(steps, page) + 3 * page,
                                   max_requests=14, num_cuda_graphs=3)
    assert engine.graphs is not None and sorted(engine.graphs.buckets) == [1, 8, 14]
    assert engine.graphs.padded_replays >= 10
    got = H.collect(steps, outputs)
    H.compare(model_dir, reqs, got, dtype)
    assert engine.cache.n_live == 0


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_d"])
def test_a_wrong_page_breaks_the_comparison(tmp_path, name, dtype):
    """The negative control of the comparisons: the mixed replay with ONE block-table entry of
    one live request pointing at another request's page, for one step, must not pass."""
    model_dir = H.make_model_dir(tmp_path, name)
    reqs = _requests(name, LENGTHS[name] + [48, 17, 80], 200)
    page = PAGES[name]
    steps = H.plan_mixed(reqs, seed=5)
    done, undo = [], []

    def swap_one_entry(engine, st):
        while undo:  # the step after: the right page is back
            slot, lp, page_id = undo.pop()
            engine.cache.groups[0].device_table[slot, lp] = page_id
        if done or len(engine.cache._requests) < 2:
            return
        engine.cache.flush_tables()
        a, b = list(engine.cache._requests.values())[:2]
        grp = engine.cache.groups[0]
        if not a.pages[0] or not b.pages[0] or a.length < page or all(e["id"] != a.request_id for e in st["entries"]):
            return
        # request a's first page becomes request b's first page on the device, for this step
        lp_a, lp_b = min(a.pages[0]), min(b.pages[0])
        grp.device_table[a.slot, lp_a] = int(b.pages[0][lp_b])
        undo.append((a.slot, lp_a, int(a.pages[0][lp_a])))
        done.append(st["step"])

    outputs, _ = H.run_engine(model_dir, dtype, steps, page, H.max_live_tokens(steps, page), before_step=swap_one_entry)
    assert done, "the control never swapped a page"
    got = H.collect(steps, outputs)
    H.record_ratios = False
    try:
        with pytest.raises(AssertionError):
            H.compare(model_dir, reqs, got, dtype)
    finally:
        H.record_ratios = True


# hidden, feed-forward, vocabulary, query heads, key/value heads, head size: widths that are odd, no
# multiple of 4 or of 8, a vocabulary of 7, groups of 5 heads, and head sizes between and beyond
# those of the tiny configurations (each has its own attention library)
ODD_SIZES = [(257, 129, 1001, 5, 1, 64), (90, 66, 97, 4, 2, 32), (100, 70, 101, 2, 1, 16), (36, 20, 7, 1, 1, 128),
             (136, 200, 211, 3, 1, 80), (136, 200, 211, 3, 1, 160), (136, 200, 211, 3, 1, 256)]


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("sizes", ODD_SIZES, ids=lambda s: "x".join(map(str, s)))
def test_replay_at_odd_sizes(tmp_path, sizes, dtype):
    """Kernels take every size a configuration allows, or refuse it with an error: never a wrong
    result.  Mixed replay with reused pages, as above."""
    from fastgen_b200.weights import write_random_model

    hidden, ffn, vocab, hq, hkv, hd = sizes
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=hidden, intermediate_size=ffn, num_hidden_layers=2,
               num_attention_heads=hq, num_key_value_heads=hkv, head_dim=hd, rms_norm_eps=1e-5, vocab_size=vocab,
               tie_word_embeddings=bool(hidden % 4), rope_theta=10000.0, max_position_embeddings=300)
    model_dir = write_random_model(tmp_path / "odd", cfg, seed=hidden + hd, norm_jitter=0.1)
    reqs = {f"r{i}": H.random_tokens(vocab, n, hidden + i) for i, n in enumerate([5, 150, 260, 64, 33])}
    steps = H.plan_mixed(reqs, seed=3)
    outputs, engine = H.run_engine(model_dir, dtype, steps, 8, H.max_live_tokens(steps, 8))
    H.compare(model_dir, reqs, H.collect(steps, outputs), dtype)
    assert engine.cache.n_live == 0


@pytest.mark.parametrize("dtype,name,page", [("float32", "tiny_b", None), ("bfloat16", "tiny_b", None),
                                             ("bfloat16", "tiny_d", 256), ("float32", "tiny_d", 48)])
def test_trace_run_program(tmp_path, dtype, name, page):
    """The same through bin/trace_run, as a user runs it: with its default page, with pages of
    256 tokens and with pages that do not divide 64 (--max-tokens still counts in 64s)."""
    model_dir = H.make_model_dir(tmp_path, name)
    reqs = _requests(name, [9, 40, 100, 64, 33], 300)
    steps = H.plan_mixed(reqs, seed=11)
    out = tmp_path / "out"
    root = Path(__file__).resolve().parent.parent
    proc = subprocess.run(
        [sys.executable, str(root / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
         "--out", str(out), "--max-tokens", str(H.max_live_tokens(steps, 64))]
        + (["--page-size", str(page)] if page else []),
        input="".join(json.dumps(s) + "\n" for s in steps), text=True, capture_output=True, timeout=900,
    )
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    vocab = H.CONFIGS[name][0]["vocab_size"]
    outputs = {s["step"]: np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab) for s in steps}
    got = H.collect(steps, outputs)
    H.compare(model_dir, reqs, got, torch.float32 if dtype == "float32" else torch.bfloat16)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["tiny_b", "tiny_d"])
@pytest.mark.parametrize("max_requests,num_graphs", [(3, 16), (12, 3)], ids=["exact", "padded"])
def test_nothing_is_written_outside_the_fed_positions(tmp_path, name, dtype, max_requests, num_graphs):
    """Every slot of every page starts as a sentinel; after a prompt in portions and some
    single tokens, only the slots of the request's own positions have changed, in its own
    pages.  "padded": 12 slots and 3 graph buckets (1, 6, 12), so the steps of two single
    tokens replay the graph of 6 lanes, four of them padding (slot -1)."""
    from fastgen_b200.engine import Engine, Model, StepEntry

    model = Model.load(H.make_model_dir(tmp_path, name), dtype, "cuda:0")
    page = PAGES[name]
    engine = Engine(model, page_size=page, n_pages=12, max_requests=max_requests, max_length=12 * page,
                    num_cuda_graphs=num_graphs)
    sentinel = 12345.0
    for grp in engine.cache.groups:
        grp.k_pages.fill_(sentinel)
        grp.v_pages.fill_(sentinel)
    vocab = H.CONFIGS[name][0]["vocab_size"]
    toks = H.random_tokens(vocab, 2 * page + 5, 8)
    engine.admit("a")
    engine.admit("idle")  # a live request that brings nothing: its slot has no pages
    cut = page + 3
    engine.step([StepEntry("a", toks[:cut], [])])
    engine.step([StepEntry("a", toks[cut:-4], [len(toks) - 4 - cut - 1])])
    padded = max_requests > 3
    other = H.random_tokens(vocab, page + 6, 9)
    if padded:
        engine.admit("b")
        engine.step([StepEntry("b", other[:-4], [])])
    for i, t in enumerate(toks[-4:]):
        entries = [StepEntry("a", [t], [0])]
        if padded:
            entries.append(StepEntry("b", [other[len(other) - 4 + i]], [0]))
        engine.step(entries)
    engine.ops.check_status()
    if padded:
        assert sorted(engine.graphs.buckets) == [6] and engine.graphs.padded_replays == 4
    lengths = {"a": len(toks), "b": len(other)} if padded else {"a": len(toks)}
    for gi, grp in enumerate(engine.cache.groups):
        owner = {}
        for rid, n in lengths.items():
            req = engine.cache.get(rid)
            assert req.length == n
            for lp, pg in req.pages[gi].items():
                owner[pg] = (lp, n)
        for pool in (grp.k_pages, grp.v_pages):  # [runs, pages, kv heads, page, head_dim]
            touched = (pool != sentinel).any(-1).any(2).any(0).cpu()  # [pages, page]
            for pg in range(pool.shape[1]):
                for slot in range(page):
                    expect = pg in owner and owner[pg][0] * page + slot < owner[pg][1]
                    assert bool(touched[pg, slot]) == expect, (gi, pg, slot)
