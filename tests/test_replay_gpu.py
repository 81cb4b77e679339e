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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    """The same through bin/trace_run, as a user runs it."""
    name = "tiny_b"
    model_dir = H.make_model_dir(tmp_path, name)
    reqs = _requests(name, [9, 40, 100, 64, 33], 300)
    steps = H.plan_mixed(reqs, seed=11)
    out = tmp_path / "out"
    root = Path(__file__).resolve().parent.parent
    proc = subprocess.run(
        [sys.executable, str(root / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
         "--out", str(out), "--max-tokens", str(H.max_live_tokens(steps, 64))],
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
def test_nothing_is_written_outside_the_fed_positions(tmp_path, name, dtype):
    """Every slot of every page starts as a sentinel; after a prompt in portions and some
    single tokens (captured graphs with padding lanes included), only the slots of the
    request's own positions have changed, in its own pages."""
    from fastgen_b200.engine import Engine, Model, StepEntry

    model = Model.load(H.make_model_dir(tmp_path, name), dtype, "cuda:0")
    page = PAGES[name]
    engine = Engine(model, page_size=page, n_pages=12, max_requests=3, max_length=12 * page)
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
    for t in toks[-4:]:
        engine.step([StepEntry("a", [t], [0])])
    engine.ops.check_status()
    req = engine.cache.get("a")
    assert req.length == len(toks)
    for gi, grp in enumerate(engine.cache.groups):
        own = req.pages[gi]
        for pool in (grp.k_pages, grp.v_pages):  # [runs, pages, kv heads, page, head_dim]
            touched = (pool != sentinel).any(-1).any(2).any(0).cpu()  # [pages, page]
            for pg in range(pool.shape[1]):
                logical = [lp for lp, p in own.items() if p == pg]
                for slot in range(page):
                    expect = bool(logical) and logical[0] * page + slot < len(toks)
                    assert bool(touched[pg, slot]) == expect, (gi, pg, slot)
