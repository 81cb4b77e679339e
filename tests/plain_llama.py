"""A plain, slow Llama decoder: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite.  It shares no code with the
``fastgen_b200`` package: it parses ``config.json`` and reads the safetensors
file on its own, and every function restates one formula of the reference
(facebookresearch/fastgen), cited as ``file:line`` within that project.

It was compared once with the reference's own model code on the CPU (see
``tests/golden/make_golden.py`` and ``tests/test_plain_vs_golden.py``).

Everything is computed in one floating-point type (float64 by default, so that
the oracle's own rounding is far below the tolerances used against it).
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Optional

import torch
from safetensors import safe_open


@dataclass
class PlainModel:
    config: dict
    weights: dict  # checkpoint tensor name -> tensor (float), q/k rows permuted
    dtype: torch.dtype

    @property
    def n_layers(self) -> int:
        return self.config["num_hidden_layers"]

    @property
    def n_heads(self) -> int:
        return self.config["num_attention_heads"]

    @property
    def n_kv_heads(self) -> int:
        # fastgen/utils/loading.py:64-67
        return self.config.get("num_key_value_heads", self.n_heads)

    @property
    def head_dim(self) -> int:
        # fastgen/model.py:54 and forward.py:364 use dim // n_heads.  A config
        # that spells head_dim out must agree with that or state its own.
        return self.config.get("head_dim") or (
            self.config["hidden_size"] // self.n_heads
        )


def permute_qk_rows(w: torch.Tensor, n_heads: int) -> torch.Tensor:
    """fastgen/utils/loading.py:296-305: within each head, new row 2j is old row
    j and new row 2j+1 is old row j + head_dim/2 (checkpoint "rotate-half" order
    -> adjacent-pair order)."""
    rows, cols = w.shape
    hd = rows // n_heads
    out = torch.empty_like(w)
    for h in range(n_heads):
        for j in range(hd // 2):
            out[h * hd + 2 * j] = w[h * hd + j]
            out[h * hd + 2 * j + 1] = w[h * hd + j + hd // 2]
    return out


def read_model(model_dir, dtype: torch.dtype = torch.float64) -> PlainModel:
    """Read ``config.json`` and ``model.safetensors`` of a model folder."""
    model_dir = Path(model_dir)
    with open(model_dir / "config.json") as f:
        config = json.load(f)
    weights = {}
    with safe_open(str(model_dir / "model.safetensors"), framework="pt", device="cpu") as f:
        for key in f.keys():
            weights[key] = f.get_tensor(key).to(dtype)
    model = PlainModel(config, weights, dtype)
    for i in range(model.n_layers):
        q = f"model.layers.{i}.self_attn.q_proj.weight"
        k = f"model.layers.{i}.self_attn.k_proj.weight"
        weights[q] = permute_qk_rows(weights[q], model.n_heads)
        weights[k] = permute_qk_rows(weights[k], model.n_kv_heads)
    return model


def rope_freqs(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """fastgen/forward.py:609-635.  The table is float32 in the reference; the
    branch conditions and the arithmetic are restated element by element."""
    pows = torch.arange(0, head_dim, 2).float() / head_dim  # forward.py:613
    freqs = 1.0 / (theta**pows)  # forward.py:614
    if not scaling:  # forward.py:616 / loading.py:75
        return freqs
    low = scaling["low_freq_factor"]
    high = scaling["high_freq_factor"]
    old_ctx = scaling["original_max_position_embeddings"]
    factor = scaling["factor"]
    low_freq_wavelen = old_ctx / low  # forward.py:622
    high_freq_wavelen = old_ctx / high  # forward.py:623
    out = freqs.clone()
    for idx in range(freqs.numel()):
        freq = freqs[idx]
        wavelen = 2 * math.pi / freq  # forward.py:627
        if wavelen > low_freq_wavelen:  # forward.py:628-629
            out[idx] = freq / factor
        if high_freq_wavelen <= wavelen <= low_freq_wavelen:  # forward.py:630-633
            x = old_ctx / wavelen - low
            x = x / (high - low)
            out[idx] = (1 - x) * freq / factor + x * freq
    return out


def embedding(table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """fastgen/forward.py:403-410: a row gather."""
    return table[tokens.long()]


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """fastgen/kernels/rmsnorm.py:33-60: x * rsqrt(sum(x^2)/D + eps) * w."""
    d = x.shape[-1]
    rstd = torch.rsqrt((x * x).sum(-1, keepdim=True) / d + eps)
    return x * rstd * w


def apply_rope(x: torch.Tensor, pos: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """fastgen/kernels/rope.py:57-89: x is [T, H, hd]; pair j of a head is
    (x[2j], x[2j+1]); angle = pos * freqs[j]."""
    # the angle is a float32 product in the reference (rope.py:57-59)
    angles = (pos.to(torch.float32)[:, None] * freqs.float()[None, :]).to(x.dtype)
    cos = torch.cos(angles)[:, None, :]
    sin = torch.sin(angles)[:, None, :]
    re = x[..., 0::2]
    im = x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = re * cos - im * sin
    out[..., 1::2] = im * cos + re * sin
    return out


def causal_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    scale: float,
    window: Optional[int] = None,
) -> torch.Tensor:
    """fastgen/forward.py:176-258 (arguments: softmax_scale = hd**-0.5, causal,
    no window, no softcap): q [T, Hq, hd], k/v [T, Hkv, hd]; query head h uses
    kv head h // (Hq/Hkv); query i sees keys j <= i (and j > i - window)."""
    t, hq, hd = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    out = torch.empty_like(q)
    idx = torch.arange(t)
    mask = idx[None, :] <= idx[:, None]
    if window is not None:
        mask = mask & (idx[None, :] > idx[:, None] - window)
    for h in range(hq):
        g = h // group
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, g, :]
    return out


def swiglu(x, w1, w3, w2):
    """fastgen/forward.py:491-496: w2(silu(w1 x) * w3 x), silu(z) = z*sigmoid(z)."""
    x1 = x @ w1.T
    x3 = x @ w3.T
    return (x1 * torch.sigmoid(x1) * x3) @ w2.T


def attention_block(m: PlainModel, i: int, a: torch.Tensor, pos: torch.Tensor, freqs):
    """fastgen/forward.py:438-470 without the cache: project, rotate q and k,
    attend, project out."""
    p = f"model.layers.{i}.self_attn."
    hd = m.head_dim
    t = a.shape[0]
    xq = (a @ m.weights[p + "q_proj.weight"].T).view(t, m.n_heads, hd)
    xk = (a @ m.weights[p + "k_proj.weight"].T).view(t, m.n_kv_heads, hd)
    xv = (a @ m.weights[p + "v_proj.weight"].T).view(t, m.n_kv_heads, hd)
    xq = apply_rope(xq, pos, freqs)
    xk = apply_rope(xk, pos, freqs)
    o = causal_attention(xq, xk, xv, hd**-0.5, m.config.get("sliding_window"))
    return o.reshape(t, m.n_heads * hd) @ m.weights[p + "o_proj.weight"].T


def forward(m: PlainModel, tokens) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence (fastgen/forward.py:347-515)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    t = tokens.numel()
    w = m.weights
    eps = m.config["rms_norm_eps"]
    freqs = rope_freqs(m.head_dim, m.config["rope_theta"], m.config.get("rope_scaling"))
    pos = torch.arange(t)
    h = embedding(w["model.embed_tokens.weight"], tokens)
    for i in range(m.n_layers):
        p = f"model.layers.{i}."
        a = rmsnorm(h, w[p + "input_layernorm.weight"], eps)  # forward.py:419
        h = h + attention_block(m, i, a, pos, freqs)  # forward.py:470-472
        f = rmsnorm(h, w[p + "post_attention_layernorm.weight"], eps)  # forward.py:474
        h = h + swiglu(  # forward.py:491-499
            f,
            w[p + "mlp.gate_proj.weight"],
            w[p + "mlp.up_proj.weight"],
            w[p + "mlp.down_proj.weight"],
        )
    h = rmsnorm(h, w["model.norm.weight"], eps)  # forward.py:501
    if m.config["tie_word_embeddings"]:  # forward.py:508-512
        out = w["model.embed_tokens.weight"]
    else:
        out = w["lm_head.weight"]
    return (h @ out.T).float()


def greedy(m: PlainModel, prompt, n_new: int) -> list[int]:
    """Greedy continuation: argmax of the last logits (generate.py:895-896),
    recomputing the whole sequence for every token."""
    seq = list(prompt)
    out = []
    for _ in range(n_new):
        tok = int(torch.argmax(forward(m, seq)[-1]))
        out.append(tok)
        seq.append(tok)
    return out


def softmax_temperature(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """fastgen/generate.py:893: softmax(logits / T)."""
    return torch.softmax(logits.double() / temperature, dim=-1)


def top_p_keep(probs: torch.Tensor, p: float) -> torch.Tensor:
    """fastgen/utils/sampling.py:26-28: in descending order, a token is dropped
    when the mass *before* it exceeds p.  Returns the boolean keep-mask in
    vocabulary order."""
    srt, idx = torch.sort(probs, dim=-1, descending=True)
    before = torch.cumsum(srt, dim=-1) - srt
    keep_sorted = ~(before > p)
    keep = torch.zeros_like(keep_sorted)
    keep.scatter_(-1, idx, keep_sorted)
    return keep
