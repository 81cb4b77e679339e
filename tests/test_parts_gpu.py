"""Each part alone against the plain implementation; a toy architecture with a
stateful mixer, registered from here without touching the package; long decoding;
first tokens; the 8B layer shape."""

import json
import math
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import helpers as H
import plain_llama as pl
from fastgen_b200.config import LayerSpec, ModelArgs, PartSpec, ScheduleEntry, register_architecture
from fastgen_b200.parts import (
    AttentionParams, Block, CacheSpec, FeedForward, Llama3Scaling, Mixer, NoPositionParams, Norm, PositionEncoding,
    RMSNormParams, RopeParams, StateSpec, SwiGLUParams, WeightSpec, make_feed_forward, make_mixer, make_norm,
    make_position, register_block, register_feed_forward, register_mixer, register_norm, register_position,
)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ops(dtype):
    from fastgen_b200.csrc.ops import Ops
    return Ops(dtype, DEV)


def _tol(dtype):
    return dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    ops = _ops(dtype)
    g = torch.Generator().manual_seed(0)
    norm = make_norm(PartSpec("rmsnorm", RMSNormParams(200, 3e-6), {"weight": "w"}))
    assert [(s.name, s.shape) for s in norm.weight_specs()] == [("w", (200,))]
    w = (1 + 0.1 * torch.randn(200, generator=g)).to(DEV, torch.bfloat16)
    norm.bind({"weight": w}, ops)
    h = torch.randn(5, 200, generator=g).to(DEV)
    d = torch.randn(5, 200, generator=g).to(DEV, dtype)
    ref = pl.rmsnorm(h.double() + d.double(), w.double(), 3e-6)
    out = norm.add_forward(h, d)
    assert out.dtype == dtype and torch.allclose(out.double(), ref, **_tol(dtype))
    assert torch.allclose(norm.forward(h).double(), ref, **_tol(dtype))  # h now holds the sum


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    ops = _ops(dtype)
    g = torch.Generator().manual_seed(1)
    ffn = make_feed_forward(PartSpec("swiglu", SwiGLUParams(72, 200), {"w1": "a", "w3": "b", "w2": "c"}))
    assert {(s.name, s.shape) for s in ffn.weight_specs()} == {("a", (200, 72)), ("b", (200, 72)), ("c", (72, 200))}
    t = {k: (torch.randn(*s, generator=g) * 0.2).to(DEV, torch.bfloat16)
         for k, s in (("w1", (200, 72)), ("w3", (200, 72)), ("w2", (72, 200)))}
    ffn.bind(t, ops)
    x = torch.randn(9, 72, generator=g).to(DEV, dtype)
    ref = pl.swiglu(x.double(), t["w1"].double(), t["w3"].double(), t["w2"].double())
    assert torch.allclose(ffn.forward(x, None).double(), ref, **_tol(dtype))


def test_position_parts():
    rope = make_position(PartSpec("rope", RopeParams(64, 500000.0, Llama3Scaling(8.0, 1.0, 4.0, 64))))
    ref = pl.rope_freqs(64, 500000.0, dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                           original_max_position_embeddings=64))
    assert torch.equal(rope.table(DEV).cpu(), ref)
    assert make_position(PartSpec("none", NoPositionParams())).table(DEV) is None


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("position,layout", [("rope", "half_split"), ("rope", "adjacent"), ("none", "adjacent")])
def test_attention_part(dtype, position, layout):
    """The mixer alone: a prompt portion, then single tokens, through a cache of its own; with
    the query and key rows in the checkpoint's half-split order (reordered at bind time) and
    in the kernels' adjacent-pair order (taken as stored)."""
    from fastgen_b200.cache import CacheManager
    from fastgen_b200.engine.step import StepContext

    ops = _ops(dtype)
    g = torch.Generator().manual_seed(2)
    dim, hq, hkv, hd, window = 72, 6, 2, 16, 20
    pos_spec = (PartSpec("rope", RopeParams(hd, 10000.0)) if position == "rope"
                else PartSpec("none", NoPositionParams()))
    spec = PartSpec("gqa_attention", AttentionParams(dim, hq, hkv, hd, pos_spec, window, qk_layout=layout),
                    {"wq": "q", "wk": "k", "wv": "v", "wo": "o"})
    mixer = make_mixer(spec)
    assert mixer.cache_spec() == CacheSpec(hkv, hd, window) and mixer.state_spec() is None
    w = {k: (torch.randn(*s, generator=g) * 0.3).to(torch.bfloat16)
         for k, s in (("wq", (hq * hd, dim)), ("wk", (hkv * hd, dim)), ("wv", (hkv * hd, dim)), ("wo", (dim, hq * hd)))}
    mixer.bind({k: v.to(DEV) for k, v in w.items()}, ops)
    cache = CacheManager([mixer.cache_spec()], [None], [None], 8, 12, 2, 96, dtype=dtype, device=DEV,
                         tensor_map_factory=ops.make_kv_tensor_maps)
    x = torch.randn(50, dim, generator=g).to(dtype)
    # plain: project, rotate, attend over the whole sequence
    xd = x.double()
    reorder = pl.permute_qk_rows if layout == "half_split" else (lambda m, heads: m)
    q = (xd @ reorder(w["wq"].double(), hq).T).view(50, hq, hd)
    k = (xd @ reorder(w["wk"].double(), hkv).T).view(50, hkv, hd)
    v = (xd @ w["wv"].double().T).view(50, hkv, hd)
    if position == "rope":
        freqs = pl.rope_freqs(hd, 10000.0, None)
        q, k = pl.apply_rope(q, torch.arange(50), freqs), pl.apply_rope(k, torch.arange(50), freqs)
    ref = pl.causal_attention(q, k, v, hd ** -0.5, window).reshape(50, hq * hd) @ w["wo"].double().T
    req = cache.admit("r")
    outs, start = [], 0
    for n in (30, 1, 1, 7, 1, 10):
        cache.reserve(req, start + n)
        cache.flush_tables()
        ctx = StepContext(DEV)
        ctx.host_seq_slot, ctx.host_seq_cached, ctx.host_seq_start = [req.slot], [start], [0, n]
        ctx.pos = torch.arange(start, start + n, dtype=torch.int32, device=DEV)
        ctx.req = torch.full((n,), req.slot, dtype=torch.int32, device=DEV)
        ctx.n_tokens = n
        outs.append(mixer.forward(x[start:start + n].to(DEV), ctx, cache.memory(0)))
        cache.advance(req, start + n)
        start += n
    ops.check_status()
    out = torch.cat(outs).double().cpu()
    # errors are measured against the outputs' scale (|y| is about 10 here): float32
    # rounding of sums of that size is about 1e-6 of it
    scale = float(ref.abs().max())
    err = float((out - ref).abs().max())
    assert err <= (1e-5 if dtype == torch.float32 else 2e-2) * scale, (err, scale)
    assert len(req.pages[0]) <= 4  # the window gave pages back


# ---------------------------------------------------------------------------------
# a toy architecture: a mixer with state of its own, a layer that runs twice, and a
# run that reads another run's cache
# ---------------------------------------------------------------------------------
@dataclass(frozen=True)
class RunningMeanParams:
    dim: int


class RunningMeanMixer(Mixer):
    """y_t = W * mean(x_0 .. x_t).  State per request: the running sum and the count."""

    def weight_specs(self):
        d = self.params.dim
        return [WeightSpec(self.names["w"], (d, d), ("normal", 0.2))]

    def state_spec(self):
        return StateSpec((self.params.dim + 1,))

    def bind(self, tensors, ops):
        self.ops = ops
        self.w = tensors["w"].float()

    def forward(self, x, ctx, memory):
        d = self.params.dim
        out = torch.empty(x.shape[0], d, dtype=torch.float32, device=x.device)
        for b, slot in enumerate(ctx.host_seq_slot):
            s, e = ctx.host_seq_start[b], ctx.host_seq_start[b + 1]
            state = memory.state[slot]
            sums = torch.cumsum(x[s:e].float(), 0) + state[:d]
            counts = state[d] + torch.arange(1, e - s + 1, device=x.device, dtype=torch.float32)
            out[s:e] = (sums / counts[:, None]) @ self.w.T
            state[:d] = sums[-1]
            state[d] = counts[-1]
        return out.to(x.dtype)


def _toy_args(cfg):
    d, v = cfg["hidden_size"], cfg["vocab_size"]
    att = AttentionParams(d, 4, 2, 16, PartSpec("rope", RopeParams(16, 10000.0)), qk_layout="half_split")

    def norm(name):
        return PartSpec("rmsnorm", RMSNormParams(d, 1e-5), {"weight": name})

    def ffn(i):
        return PartSpec("swiglu", SwiGLUParams(d, 96), {"w1": f"l{i}.w1", "w3": f"l{i}.w3", "w2": f"l{i}.w2"})

    def attn(i):
        return PartSpec("gqa_attention", att, {"wq": f"l{i}.q", "wk": f"l{i}.k", "wv": f"l{i}.v", "wo": f"l{i}.o"})

    layers = [
        LayerSpec("prenorm", PartSpec("running_mean", RunningMeanParams(d), {"w": "l0.mix"}), norm("l0.n1"), ffn(0), norm("l0.n2")),
        LayerSpec("prenorm", attn(1), norm("l1.n1"), ffn(1), norm("l1.n2")),
        LayerSpec("prenorm", attn(2), norm("l2.n1"), ffn(2), norm("l2.n2")),
    ]
    # layer 0 runs twice (two states), layer 2 reads the cache layer 1's run wrote
    schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(2, kv_from=1)]
    return ModelArgs("ToyForCausalLM", d, v, cfg["max_position_embeddings"], False, "emb", "out",
                     tuple(layers), tuple(schedule), norm("final"))


def _toy_plain(w, tokens):
    """The toy model, whole sequence, float64."""
    def block_ffn(h, i):
        f = pl.rmsnorm(h, w[f"l{i}.n2"], 1e-5)
        return h + pl.swiglu(f, w[f"l{i}.w1"], w[f"l{i}.w3"], w[f"l{i}.w2"])

    def mean_layer(h):
        a = pl.rmsnorm(h, w["l0.n1"], 1e-5)
        cm = torch.cumsum(a, 0) / torch.arange(1, a.shape[0] + 1, dtype=a.dtype)[:, None]
        return block_ffn(h + cm @ w["l0.mix"].T, 0)

    t = len(tokens)
    freqs = pl.rope_freqs(16, 10000.0, None)
    pos = torch.arange(t)
    h = w["emb"][torch.tensor(tokens)]
    h = mean_layer(h)
    a = pl.rmsnorm(h, w["l1.n1"], 1e-5)
    k = pl.apply_rope((a @ pl.permute_qk_rows(w["l1.k"], 2).T).view(t, 2, 16), pos, freqs)
    v = (a @ w["l1.v"].T).view(t, 2, 16)
    q = pl.apply_rope((a @ pl.permute_qk_rows(w["l1.q"], 4).T).view(t, 4, 16), pos, freqs)
    h = block_ffn(h + pl.causal_attention(q, k, v, 0.25).reshape(t, 64) @ w["l1.o"].T, 1)
    h = mean_layer(h)
    a = pl.rmsnorm(h, w["l2.n1"], 1e-5)
    q = pl.apply_rope((a @ pl.permute_qk_rows(w["l2.q"], 4).T).view(t, 4, 16), pos, freqs)
    h = block_ffn(h + pl.causal_attention(q, k, v, 0.25).reshape(t, 64) @ w["l2.o"].T, 2)  # layer 1's keys and values
    return pl.rmsnorm(h, w["final"], 1e-5) @ w["out"].T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_architecture_with_stateful_mixer(tmp_path, dtype):
    from safetensors.torch import load_file
    from fastgen_b200.weights import write_random_model

    register_mixer("running_mean", RunningMeanMixer)
    register_architecture("ToyForCausalLM", _toy_args)
    cfg = dict(architectures=["ToyForCausalLM"], hidden_size=64, vocab_size=97, max_position_embeddings=256)
    model_dir = write_random_model(tmp_path / "toy", cfg, seed=11, norm_jitter=0.1, std=0.1)
    w = {k: v.double() for k, v in load_file(str(model_dir / "model.safetensors")).items()}
    reqs = {f"t{i}": H.random_tokens(97, n, 40 + i) for i, n in enumerate([9, 33, 50, 21, 40, 12])}
    steps = H.plan_mixed(reqs, seed=3, max_live=3)
    outputs, engine = H.run_engine(model_dir, dtype, steps, page_size=8,
                                   max_tokens=H.max_live_tokens(steps, 8), max_requests=3)
    assert engine.graphs is None  # a mixer that does not declare itself graph-safe is never captured
    assert len(engine.cache.groups) == 1 and engine.cache.groups[0].entries == [1]
    assert [s is not None for s in engine.cache.states] == [True, False, True, False]
    got = H.collect(steps, outputs)
    for rid, toks in reqs.items():
        ref = _toy_plain(w, toks).numpy()
        for p, row in got[rid].items():
            H.check_row(row, ref[p], dtype, f"{rid} pos {p}")


# ---------------------------------------------------------------------------------
# a second toy architecture: a feed-forward with routing, a position encoding of its own,
# a norm of its own and another arrangement of the block, all registered from here
# ---------------------------------------------------------------------------------
@dataclass(frozen=True)
class RoutedParams:
    dim: int
    ffn_dim: int
    n_experts: int


class RoutedFeedForward(FeedForward):
    """y = sum_e softmax(x R^T)_e * W2_e relu(W1_e x): router logits and weights in float32."""

    def weight_specs(self):
        p = self.params
        return [WeightSpec(self.names["router"], (p.n_experts, p.dim), ("normal", 0.3)),
                WeightSpec(self.names["w1"], (p.n_experts, p.ffn_dim, p.dim), ("normal", 0.1)),
                WeightSpec(self.names["w2"], (p.n_experts, p.dim, p.ffn_dim), ("normal", 0.1))]

    def bind(self, tensors, ops):
        self.router, self.w1, self.w2 = (tensors[k].float() for k in ("router", "w1", "w2"))

    def forward(self, x, ctx):
        xf = x.float()
        gate = torch.softmax(xf @ self.router.T, -1)
        y = torch.zeros_like(xf)
        for e in range(self.params.n_experts):
            y += gate[:, e:e + 1] * (torch.relu(xf @ self.w1[e].T) @ self.w2[e].T)
        return y.to(x.dtype)


@dataclass(frozen=True)
class PartialRopeParams:
    head_dim: int
    theta: float
    rotated_pairs: int  # the first pairs are rotated, the rest are left as they are


class PartialRope(PositionEncoding):
    def table(self, device):
        p = self.params
        j = torch.arange(p.head_dim // 2, dtype=torch.float32)
        freqs = p.theta ** (-2.0 * j / (2 * p.rotated_pairs))
        freqs[p.rotated_pairs:] = 0.0  # angle 0: not rotated
        return freqs.to(device)


class ToyLayerNorm(Norm):
    """(x - mean) / sqrt(var + eps) * w, float32 arithmetic."""

    def weight_specs(self):
        return [WeightSpec(self.names["weight"], (self.params.dim,), ("ones",))]

    def bind(self, tensors, ops):
        self.ops = ops
        self.weight = tensors["weight"].float()

    def forward(self, x, out_dtype=None, rows=None):
        xf = x.float() if rows is None else x.float()[rows.long()]
        y = (xf - xf.mean(-1, keepdim=True)) * torch.rsqrt(xf.var(-1, unbiased=False, keepdim=True) + self.params.eps)
        return (y * self.weight).to(out_dtype or self.ops.act_dtype)


class ParallelBlock(Block):
    """h = h + mixer(norm(h)) + ffn(norm(h)): one norm, both parts read it."""

    def forward(self, h, pending, ctx, memory):
        if pending is not None:
            h.add_(pending.float())
        a = self.mixer_norm.forward(h)
        return h, self.mixer.forward(a, ctx, memory).float() + self.ffn.forward(a, ctx).float()


def _toy2_args(cfg):
    d, v = cfg["hidden_size"], cfg["vocab_size"]

    def attn(i, position):
        return PartSpec("gqa_attention", AttentionParams(d, 3, 3, 16, position),
                        {"wq": f"l{i}.q", "wk": f"l{i}.k", "wv": f"l{i}.v", "wo": f"l{i}.o"})

    ln = lambda name: PartSpec("toy_layernorm", RMSNormParams(d, 1e-3), {"weight": name})
    rms = lambda name: PartSpec("rmsnorm", RMSNormParams(d, 1e-5), {"weight": name})
    routed = PartSpec("toy_routed", RoutedParams(d, 40, 3), {"router": "l0.r", "w1": "l0.e1", "w2": "l0.e2"})
    swiglu = PartSpec("swiglu", SwiGLUParams(d, 72), {"w1": "l1.w1", "w3": "l1.w3", "w2": "l1.w2"})
    layers = (
        LayerSpec("toy_parallel", attn(0, PartSpec("toy_partial_rope", PartialRopeParams(16, 100.0, 5))), ln("l0.n"),
                  routed, ln("l0.n")),
        LayerSpec("prenorm", attn(1, PartSpec("none", NoPositionParams())), rms("l1.n1"), swiglu, rms("l1.n2")),
    )
    return ModelArgs("Toy2ForCausalLM", d, v, cfg["max_position_embeddings"], False, "emb", "out", layers,
                     (ScheduleEntry(0), ScheduleEntry(1)), rms("final"))


def _toy2_plain(w, tokens):
    t = len(tokens)
    pos = torch.arange(t)
    h = w["emb"][torch.tensor(tokens)]
    # layer 0: parallel block, layer norm, partial rotation, routed feed-forward
    a = (h - h.mean(-1, keepdim=True)) * torch.rsqrt(h.var(-1, unbiased=False, keepdim=True) + 1e-3) * w["l0.n"]
    j = torch.arange(8, dtype=torch.float64)
    freqs = 100.0 ** (-2.0 * j / 10)
    freqs[5:] = 0.0
    # (this toy stores its query and key rows as adjacent pairs: no reordering)
    q = pl.apply_rope((a @ w["l0.q"].T).view(t, 3, 16), pos, freqs)
    k = pl.apply_rope((a @ w["l0.k"].T).view(t, 3, 16), pos, freqs)
    v = (a @ w["l0.v"].T).view(t, 3, 16)
    mix = pl.causal_attention(q, k, v, 0.25).reshape(t, 48) @ w["l0.o"].T
    gate = torch.softmax(a @ w["l0.r"].T, -1)
    ffn = sum(gate[:, e:e + 1] * (torch.relu(a @ w["l0.e1"][e].T) @ w["l0.e2"][e].T) for e in range(3))
    h = h + mix + ffn
    # layer 1: the usual block without a position encoding
    a = pl.rmsnorm(h, w["l1.n1"], 1e-5)
    q, k, v = ((a @ w[f"l1.{n}"].T).view(t, 3, 16) for n in "qkv")
    h = h + pl.causal_attention(q, k, v, 0.25).reshape(t, 48) @ w["l1.o"].T
    h = h + pl.swiglu(pl.rmsnorm(h, w["l1.n2"], 1e-5), w["l1.w1"], w["l1.w3"], w["l1.w2"])
    return pl.rmsnorm(h, w["final"], 1e-5) @ w["out"].T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_architecture_with_routing_and_other_parts(tmp_path, dtype):
    """A feed-forward with routing, a position encoding, a norm and a block arrangement that
    the package does not have, registered here, built from a model folder and stepped in
    mixed batches, against the same model written out plainly."""
    from safetensors.torch import load_file
    from fastgen_b200.weights import write_random_model

    register_feed_forward("toy_routed", RoutedFeedForward)
    register_position("toy_partial_rope", PartialRope)
    register_norm("toy_layernorm", ToyLayerNorm)
    register_block("toy_parallel", ParallelBlock)
    register_architecture("Toy2ForCausalLM", _toy2_args)
    cfg = dict(architectures=["Toy2ForCausalLM"], hidden_size=48, vocab_size=83, max_position_embeddings=128)
    model_dir = write_random_model(tmp_path / "toy2", cfg, seed=5, norm_jitter=0.1, std=0.1)
    w = {k: v.double() for k, v in load_file(str(model_dir / "model.safetensors")).items()}
    reqs = {f"u{i}": H.random_tokens(83, n, 70 + i) for i, n in enumerate([5, 40, 17, 64, 9])}
    steps = H.plan_mixed(reqs, seed=9, max_live=3)
    outputs, engine = H.run_engine(model_dir, dtype, steps, page_size=8,
                                   max_tokens=H.max_live_tokens(steps, 8), max_requests=3)
    got = H.collect(steps, outputs)
    for rid, toks in reqs.items():
        ref = _toy2_plain(w, toks).numpy()
        for p, row in got[rid].items():
            H.check_row(row, ref[p], dtype, f"{rid} pos {p}")


# ---------------------------------------------------------------------------------
# a third toy architecture: a mixer that caches ONE compressed entry a token, in pages of a
# size of its own (a second group beside the ordinary attention's), and a block arrangement
# with six parts (norms after the mixer and after the feed-forward)
# ---------------------------------------------------------------------------------
@dataclass(frozen=True)
class LatentParams:
    dim: int
    rank: int
    page: int


class LatentAttention(Mixer):
    """One head; per token the cache holds c = Wc x (``rank`` numbers) in a single pool, and
    keys Wk c and values Wv c are made from the cached entries at every step."""

    def weight_specs(self):
        p = self.params
        return [WeightSpec(self.names[n], shape, ("normal", 0.25)) for n, shape in
                (("wc", (p.rank, p.dim)), ("wq", (p.rank, p.dim)), ("wk", (p.rank, p.rank)),
                 ("wv", (p.rank, p.rank)), ("wo", (p.dim, p.rank)))]

    def cache_spec(self):
        return CacheSpec(1, self.params.rank, None, n_pools=1, page_size=self.params.page)

    def bind(self, tensors, ops):
        self.w = {k: v.float() for k, v in tensors.items()}

    def forward(self, x, ctx, memory):
        p, w = self.params, self.w
        assert memory.v_pages is None and memory.page_size == p.page
        pool = memory.k_pages  # [pages, 1, page, rank]
        out = torch.empty(x.shape[0], p.dim, dtype=torch.float32, device=x.device)
        for b, slot in enumerate(ctx.host_seq_slot):
            s, e, cached = ctx.host_seq_start[b], ctx.host_seq_start[b + 1], ctx.host_seq_cached[b]
            xf = x[s:e].float()
            pos = torch.arange(cached, cached + e - s, device=x.device)
            row = memory.block_table[slot].long()
            pool[row[pos // p.page], 0, pos % p.page] = (xf @ w["wc"].T).to(pool.dtype)
            every = torch.arange(cached + e - s, device=x.device)
            c = pool[row[every // p.page], 0, every % p.page].float()
            scores = (xf @ w["wq"].T) @ (c @ w["wk"].T).T * p.rank ** -0.5
            scores = scores.masked_fill(every[None, :] > pos[:, None], float("-inf"))
            out[s:e] = torch.softmax(scores, -1) @ (c @ w["wv"].T) @ w["wo"].T
        return out.to(x.dtype)


class SandwichBlock(Block):
    """h += post_mixer_norm(mixer(norm(h))); h += post_ffn_norm(ffn(norm(h)))."""

    def forward(self, h, pending, ctx, memory):
        a = self.mixer_norm.add_forward(h, pending)
        m = self.extra["post_mixer_norm"].forward(self.mixer.forward(a, ctx, memory).float())
        f = self.ffn_norm.add_forward(h, m)
        return h, self.extra["post_ffn_norm"].forward(self.ffn.forward(f, ctx).float())


def _toy3_args(cfg):
    d, v = cfg["hidden_size"], cfg["vocab_size"]
    rms = lambda name: PartSpec("rmsnorm", RMSNormParams(d, 1e-5), {"weight": name})
    att = PartSpec("gqa_attention", AttentionParams(d, 2, 1, 16, PartSpec("rope", RopeParams(16, 10000.0))),
                   {"wq": "l1.q", "wk": "l1.k", "wv": "l1.v", "wo": "l1.o"})
    latent = PartSpec("toy_latent", LatentParams(d, 12, 4), {n: f"l0.{n}" for n in ("wc", "wq", "wk", "wv", "wo")})
    ffn = lambda i: PartSpec("swiglu", SwiGLUParams(d, 56), {"w1": f"l{i}.w1", "w3": f"l{i}.w3", "w2": f"l{i}.w2"})
    layers = (
        LayerSpec("toy_sandwich", latent, rms("l0.n1"), ffn(0), rms("l0.n2"),
                  extra=(("post_mixer_norm", "norm", rms("l0.n3")), ("post_ffn_norm", "norm", rms("l0.n4")))),
        LayerSpec("prenorm", att, rms("l1.n1"), ffn(1), rms("l1.n2")),
    )
    return ModelArgs("Toy3ForCausalLM", d, v, cfg["max_position_embeddings"], False, "emb", "out", layers,
                     (ScheduleEntry(0), ScheduleEntry(1)), rms("final"))


def _toy3_plain(w, tokens):
    t = len(tokens)
    h = w["emb"][torch.tensor(tokens)]
    a = pl.rmsnorm(h, w["l0.n1"], 1e-5)
    c = a @ w["l0.wc"].T
    scores = (a @ w["l0.wq"].T) @ (c @ w["l0.wk"].T).T * 12 ** -0.5
    scores = scores.masked_fill(torch.arange(t)[None, :] > torch.arange(t)[:, None], float("-inf"))
    mix = torch.softmax(scores, -1) @ (c @ w["l0.wv"].T) @ w["l0.wo"].T
    h = h + pl.rmsnorm(mix, w["l0.n3"], 1e-5)
    f = pl.swiglu(pl.rmsnorm(h, w["l0.n2"], 1e-5), w["l0.w1"], w["l0.w3"], w["l0.w2"])
    h = h + pl.rmsnorm(f, w["l0.n4"], 1e-5)
    a = pl.rmsnorm(h, w["l1.n1"], 1e-5)
    freqs = pl.rope_freqs(16, 10000.0, None)
    q = pl.apply_rope((a @ w["l1.q"].T).view(t, 2, 16), torch.arange(t), freqs)
    k = pl.apply_rope((a @ w["l1.k"].T).view(t, 1, 16), torch.arange(t), freqs)
    h = h + pl.causal_attention(q, k, (a @ w["l1.v"].T).view(t, 1, 16), 0.25).reshape(t, 32) @ w["l1.o"].T
    h = h + pl.swiglu(pl.rmsnorm(h, w["l1.n2"], 1e-5), w["l1.w1"], w["l1.w3"], w["l1.w2"])
    return pl.rmsnorm(h, w["final"], 1e-5) @ w["out"].T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_architecture_with_a_one_pool_cache_and_six_parts(tmp_path, dtype):
    """Two groups of pages with different page sizes (the latent mixer's pages of 4 entries in a
    single pool, the attention's pages of 8 keys and values), each with its own block table and
    its own free pages; a block with six parts; all registered here."""
    from safetensors.torch import load_file
    from fastgen_b200.weights import write_random_model

    register_mixer("toy_latent", LatentAttention)
    register_block("toy_sandwich", SandwichBlock)
    register_architecture("Toy3ForCausalLM", _toy3_args)
    cfg = dict(architectures=["Toy3ForCausalLM"], hidden_size=40, vocab_size=61, max_position_embeddings=96)
    model_dir = write_random_model(tmp_path / "toy3", cfg, seed=8, norm_jitter=0.1, std=0.1)
    w = {k: v.double() for k, v in load_file(str(model_dir / "model.safetensors")).items()}
    assert {"l0.n3", "l0.n4", "l0.wc"} <= set(w)  # the extra parts' tensors were declared and written
    reqs = {f"v{i}": H.random_tokens(61, n, 30 + i) for i, n in enumerate([7, 33, 18, 50, 11])}
    steps = H.plan_mixed(reqs, seed=4, max_live=3)
    outputs, engine = H.run_engine(model_dir, dtype, steps, page_size=8,
                                   max_tokens=H.max_live_tokens(steps, 8), max_requests=3)
    groups = engine.cache.groups
    assert [g.page_size for g in groups] == [4, 8] and groups[0].v_pages is None and groups[1].v_pages is not None
    assert groups[0].pool.n_pages == 2 * groups[1].pool.n_pages  # the same number of tokens
    got = H.collect(steps, outputs)
    for rid, toks in reqs.items():
        ref = _toy3_plain(w, toks).numpy()
        for p, row in got[rid].items():
            H.check_row(row, ref[p], dtype, f"{rid} pos {p}")
    assert engine.cache.free_pages() == [g.pool.n_pages for g in groups]


# ---------------------------------------------------------------------------------
# a mixer with state that may be captured in a graph: a bucket that is captured when a step
# first meets it must not advance any request's state by its warm-up run
# ---------------------------------------------------------------------------------
@dataclass(frozen=True)
class CountParams:
    dim: int


class CountingMixer(Mixer):
    """y_t = x_t * (1 + count_t / 16), count_t = tokens of the request up to and including t.
    Device-side work of fixed shape only, padding lanes (slot -1) left alone: graph-safe."""

    graph_safe = True

    def state_spec(self):
        return StateSpec((1,))

    def bind(self, tensors, ops):
        pass

    def forward(self, x, ctx, memory):
        live = ctx.req >= 0
        slot = ctx.req.clamp(min=0).long()
        # position + 1 = the count; the state keeps the last count, so a forward pass that ran
        # twice for a step would show as a count that is ahead of the position
        memory.state.index_add_(0, slot, live.to(torch.float32)[:, None])
        count = torch.where(live, memory.state[slot, 0], torch.zeros((), device=x.device))
        return (x.float() * (1 + count[:, None] / 16)).to(x.dtype)


def _count_args(cfg):
    d, v = cfg["hidden_size"], cfg["vocab_size"]
    rms = lambda name: PartSpec("rmsnorm", RMSNormParams(d, 1e-5), {"weight": name})
    ffn = PartSpec("swiglu", SwiGLUParams(d, 40), {"w1": "w1", "w3": "w3", "w2": "w2"})
    layers = (LayerSpec("prenorm", PartSpec("toy_count", CountParams(d), {}), rms("n1"), ffn, rms("n2")),)
    return ModelArgs("CountForCausalLM", d, v, cfg["max_position_embeddings"], False, "emb", "out", layers,
                     (ScheduleEntry(0),), rms("final"))


def _count_plain(w, tokens):
    h = w["emb"][torch.tensor(tokens)]
    count = torch.arange(1, len(tokens) + 1, dtype=torch.float64)
    h = h + pl.rmsnorm(h, w["n1"], 1e-5) * (1 + count[:, None] / 16)
    h = h + pl.swiglu(pl.rmsnorm(h, w["n2"], 1e-5), w["w1"], w["w3"], w["w2"])
    return pl.rmsnorm(h, w["final"], 1e-5) @ w["out"].T


def test_stateful_graph_safe_mixer_through_lazily_captured_graphs(tmp_path):
    """Single tokens only, fed one step at a time: every bucket is captured when a step first
    needs it (no capture_all), while its requests are live.  The state counts each token once."""
    from safetensors.torch import load_file
    from fastgen_b200.engine import Engine, Model, StepEntry
    from fastgen_b200.weights import write_random_model

    register_mixer("toy_count", CountingMixer)
    register_architecture("CountForCausalLM", _count_args)
    cfg = dict(architectures=["CountForCausalLM"], hidden_size=32, vocab_size=50, max_position_embeddings=64)
    model_dir = write_random_model(tmp_path / "count", cfg, seed=3, norm_jitter=0.1, std=0.2)
    w = {k: v.double() for k, v in load_file(str(model_dir / "model.safetensors")).items()}
    model = Model.load(model_dir, torch.float32, DEV)
    engine = Engine(model, page_size=8, n_pages=8, max_requests=6, num_cuda_graphs=3)
    assert engine.graphs is not None and not engine.graphs.buckets
    reqs = {f"c{i}": H.random_tokens(50, 12, 20 + i) for i in range(5)}
    for rid in reqs:
        engine.admit(rid)
    got = {rid: [] for rid in reqs}
    for t in range(12):
        # the number of requests in a step changes, so the buckets 1, 4 (3.5 rounded) and 6 are met
        # one after the other, each for the first time in the middle of the requests' lives
        ids = list(reqs)[: 1 + (t % 5)] if t >= 2 else list(reqs)
        ids = [rid for rid in ids if len(got[rid]) < 12]
        logits = engine.step([StepEntry(rid, [reqs[rid][len(got[rid])]], [0]) for rid in ids])
        for rid, row in zip(ids, logits.cpu().numpy()):
            got[rid].append(row)
    assert len(engine.graphs.buckets) >= 2 and engine.graphs.replays >= 10
    for rid, toks in reqs.items():
        n = len(got[rid])
        ref = _count_plain(w, toks[:n]).numpy()
        for p_, row in enumerate(got[rid]):
            H.check_row(row, ref[p_], torch.float32, f"{rid} pos {p_}")
        assert float(engine.cache.states[0][engine.cache.get(rid).slot, 0]) == n


# ---------------------------------------------------------------------------------
# long decoding and first tokens
# ---------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["tiny_b", "tiny_c"])
def test_long_decoding(tmp_path, name, dtype):
    """A short prompt, then hundreds of single tokens: every page edge and every edge of
    the key splits is crossed one token at a time (captured graphs included)."""
    model_dir = H.make_model_dir(tmp_path, name)
    vocab = H.CONFIGS[name][0]["vocab_size"]
    reqs = {"long": H.random_tokens(vocab, 330, 9), "other": H.random_tokens(vocab, 150, 10)}
    steps, n = [], 0
    steps.append(dict(step=n, entries=[dict(id="long", tokens=reqs["long"][:3], want=[0, 1, 2])], end=[])); n += 1
    for p in range(3, 330):
        entries = [dict(id="long", tokens=[reqs["long"][p]], want=[0])]
        q = p - 100  # a second request joins later and decodes beside the first
        if 0 <= q < 150:
            entries.append(dict(id="other", tokens=[reqs["other"][q]], want=[0]))
        steps.append(dict(step=n, entries=entries, end=[])); n += 1
    outputs, engine = H.run_engine(model_dir, dtype, steps, page_size=16, max_tokens=512)
    H.compare(model_dir, reqs, H.collect(steps, outputs), dtype)
    assert engine.graphs is not None and engine.graphs.replays >= 300


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_first_tokens(tmp_path, dtype):
    """Position 0 alone, then positions 1, 2, 3 one by one, for requests that start in different steps."""
    model_dir = H.make_model_dir(tmp_path, "tiny_a")
    reqs = {f"f{i}": H.random_tokens(256, 4, 60 + i) for i in range(3)}
    steps = []
    for s in range(6):
        entries = [dict(id=rid, tokens=[toks[s - i]], want=[0]) for i, (rid, toks) in enumerate(reqs.items())
                   if 0 <= s - i < 4]
        steps.append(dict(step=s, entries=entries, end=[]))
    outputs, _ = H.run_engine(model_dir, dtype, steps, page_size=8, max_tokens=64)
    H.compare(model_dir, reqs, H.collect(steps, outputs), dtype)


@pytest.mark.parametrize("dtype,step_graphs", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
def test_long_prompt_in_large_portions(tmp_path, dtype, step_graphs):
    """A prompt of thousands of tokens in portions of thousands (dozens of key tiles a query
    tile, llama3-scaled angles beyond the original context), then in portions of a hundred and
    of a dozen tokens on thousands of cached keys (few items with many key tiles each, which the
    bfloat16 prompt kernel works on in parts), then single tokens over dozens of key splits;
    eagerly and with the portions' steps replayed from captured graphs."""
    cfg = dict(
        architectures=["LlamaForCausalLM"], hidden_size=256, intermediate_size=344, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-5, vocab_size=300, tie_word_embeddings=False,
        rope_theta=500000.0,
        rope_scaling=dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=1024),
        max_position_embeddings=16384,
    )
    from fastgen_b200.weights import write_random_model
    model_dir = write_random_model(tmp_path / "long", cfg, seed=3, norm_jitter=0.1)
    n = 6200
    toks = H.random_tokens(300, n, 1)
    head = n - 6
    steps, p = [], 0
    for chunk in (3000, 2048, 1000, 130, 2, head - 6180):
        steps.append(dict(step=len(steps), entries=[dict(id="a", tokens=toks[p:p + chunk], want=[0, chunk // 2, chunk - 1])],
                          end=[]))
        p += chunk
    assert p == head
    for p in range(head, n):
        steps.append(dict(step=len(steps), entries=[dict(id="a", tokens=[toks[p]], want=[0])], end=[]))
    outputs, engine = H.run_engine(model_dir, dtype, steps, page_size=64, max_tokens=8192,
                                   max_step_tokens=3072 if step_graphs else None)
    if step_graphs:
        assert engine.step_graphs is not None and engine.step_graphs.replays >= 5
    if dtype == torch.bfloat16:
        # the small portions' long items were worked on in parts (the prompt kernel leaves the
        # number of parts of every item of a launch that split), from captured graphs too
        assert int(engine.ops._split[64][1][1::2].max()) >= 2
    got = H.collect(steps, outputs)["a"]
    ref = H.plain_logits(model_dir, toks)
    assert len(got) == 3 * 6 - 1 + 6  # (the portion of two tokens has two places)
    for p, row in got.items():
        H.check_row(row, ref[p], dtype, f"pos {p}")


@pytest.mark.parametrize("step_graphs", [False, True])
def test_mixed_portions_on_long_contexts(tmp_path, step_graphs):
    """Steps that mix portions of a few tokens of two requests with thousands of cached keys,
    a fresh prompt and single tokens of two more requests: few attention items of very
    different lengths in one launch (some worked on in parts, some not), eagerly and from
    captured graphs whose tile lists have padding entries in front of the real ones."""
    cfg = dict(
        architectures=["LlamaForCausalLM"], hidden_size=256, intermediate_size=344, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-5, vocab_size=300, tie_word_embeddings=False,
        rope_theta=500000.0, max_position_embeddings=8192,
    )
    from fastgen_b200.weights import write_random_model
    model_dir = write_random_model(tmp_path / "mixed_long", cfg, seed=5, norm_jitter=0.1)
    reqs = {"a": H.random_tokens(300, 3100, 1), "b": H.random_tokens(300, 1600, 2), "c": H.random_tokens(300, 90, 3),
            "d": H.random_tokens(300, 2210, 4), "e": H.random_tokens(300, 530, 5)}
    steps = []

    def step(entries, end=()):
        steps.append(dict(step=len(steps), entries=[dict(id=i, tokens=t, want=w) for i, t, w in entries], end=list(end)))

    # most of a, b, d and e, each alone
    step([("a", reqs["a"][:3000], [2999])])
    step([("b", reqs["b"][:1500], [1499])])
    step([("d", reqs["d"][:2200], [2199])])
    step([("e", reqs["e"][:520], [519])])
    # portions of a and b on their long contexts beside c's whole prompt and single tokens of d and e
    step([("a", reqs["a"][3000:3040], [0, 39]), ("d", reqs["d"][2200:2201], [0]), ("b", reqs["b"][1500:1509], [8]),
          ("c", reqs["c"][:70], [69]), ("e", reqs["e"][520:521], [0])])
    step([("e", reqs["e"][521:522], [0]), ("a", reqs["a"][3040:3042], [0, 1]), ("b", reqs["b"][1509:1600], [0, 90]),
          ("d", reqs["d"][2201:2202], [0]), ("c", reqs["c"][70:90], [19])], end=["b", "c"])
    step([("a", reqs["a"][3042:3100], [57]), ("d", reqs["d"][2202:2203], [0]), ("e", reqs["e"][522:530], [7])],
         end=["a", "d", "e"])
    outputs, engine = H.run_engine(model_dir, torch.bfloat16, steps, page_size=64, max_tokens=8192, max_requests=5,
                                   max_step_tokens=3072 if step_graphs else None)
    if step_graphs:
        assert engine.step_graphs is not None and engine.step_graphs.replays >= 6  # (the 520-token prompt is too far from its bucket and runs eagerly)
    assert int(engine.ops._split[64][1][1::2].max()) >= 2  # some items were worked on in parts
    got = H.collect(steps, outputs)
    for rid, toks in reqs.items():
        ref = H.plain_logits(model_dir, toks)
        assert got[rid], rid
        for p, row in got[rid].items():
            H.check_row(row, ref[p], torch.bfloat16, f"{rid} pos {p}")


def test_many_key_splits_through_graphs(tmp_path):
    """Four live requests with thousands of cached keys and eight key/value heads: enough
    (request, head, split) items for the persistent single-token kernel, inside captured
    graphs with programmatic dependent launch, where a load that is moved above the wait on
    the kernel before would see the step before."""
    cfg = dict(
        architectures=["LlamaForCausalLM"], hidden_size=128, intermediate_size=136, num_hidden_layers=2,
        num_attention_heads=16, num_key_value_heads=8, head_dim=64, rms_norm_eps=1e-5, vocab_size=211,
        tie_word_embeddings=False, rope_theta=10000.0, max_position_embeddings=4096,
    )
    from fastgen_b200.weights import write_random_model
    model_dir = write_random_model(tmp_path / "wide", cfg, seed=21, norm_jitter=0.1)
    lengths = [2400, 2500, 2300, 2450]
    tail = 5
    reqs = {f"w{i}": H.random_tokens(211, n, 400 + i) for i, n in enumerate(lengths)}
    steps = []
    for rid, toks in reqs.items():
        head = len(toks) - tail
        steps.append(dict(step=len(steps), entries=[dict(id=rid, tokens=toks[:head], want=[head - 1])], end=[]))
    for k in range(tail):
        entries = [dict(id=rid, tokens=[toks[len(toks) - tail + k]], want=[0]) for rid, toks in reqs.items()]
        steps.append(dict(step=len(steps), entries=entries, end=[]))
    outputs, engine = H.run_engine(model_dir, torch.bfloat16, steps, page_size=64, max_tokens=4 * 2560)
    assert engine.graphs is not None and engine.graphs.replays >= tail
    got = H.collect(steps, outputs)
    for rid, toks in reqs.items():
        ref = H.plain_logits(model_dir, toks)
        for p, row in got[rid].items():
            H.check_row(row, ref[p], torch.bfloat16, f"{rid} pos {p}")


# ---------------------------------------------------------------------------------
# the sizes of a Llama-3.1-8B layer (two layers, a small vocabulary)
# ---------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_8b_layer_shape(tmp_path, dtype):
    cfg = dict(
        architectures=["LlamaForCausalLM"], hidden_size=4096, intermediate_size=14336, num_hidden_layers=2,
        num_attention_heads=32, num_key_value_heads=8, rms_norm_eps=1e-5, vocab_size=1031,
        tie_word_embeddings=False, rope_theta=500000.0,
        rope_scaling=dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192),
        max_position_embeddings=131072,
    )
    from fastgen_b200.weights import write_random_model
    model_dir = write_random_model(tmp_path / "big", cfg, seed=4)
    toks = H.random_tokens(1031, 150, 5)
    other = H.random_tokens(1031, 70, 6)
    ref = pl.forward(pl.read_model(model_dir, torch.float64), toks).numpy()
    ref_other = pl.forward(pl.read_model(model_dir, torch.float64), other).numpy()
    steps = [
        dict(step=0, entries=[dict(id="a", tokens=toks[:100], want=list(range(100)))], end=[]),
        dict(step=1, entries=[dict(id="a", tokens=toks[100:130], want=list(range(30))),
                              dict(id="b", tokens=other[:69], want=list(range(69)))], end=[]),
    ]
    for p in range(130, 150):
        e = [dict(id="a", tokens=[toks[p]], want=[0])]
        if p == 130:
            e.append(dict(id="b", tokens=[other[69]], want=[0]))
        steps.append(dict(step=len(steps), entries=e, end=["b"] if p == 130 else []))
    outputs, _ = H.run_engine(model_dir, dtype, steps, page_size=64, max_tokens=512)
    got = H.collect(steps, outputs)
    for rows, r in ((got["a"], ref), (got["b"], ref_other)):
        for p, row in rows.items():
            H.check_row(row, r[p], dtype, f"pos {p}", wide=True)
