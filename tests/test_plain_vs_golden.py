"""The plain implementation against logits made once by the reference's own code.

``tests/golden/make_golden.py`` ran the reference's model code (Transformer,
loader, rope table, Triton kernels under the interpreter; attention replaced by
a formula shim) on the CPU in float32 and stored the logits.  The weights are
redrawn here from the same seed; a checksum guards against the writer drifting.
"""

import hashlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers as H
import plain_llama as pl

GOLDEN = Path(__file__).resolve().parent / "golden"


def _checksum(model_dir) -> str:
    from safetensors import safe_open

    h = hashlib.sha256()
    with safe_open(str(Path(model_dir) / "model.safetensors"), framework="pt", device="cpu") as f:
        for key in sorted(f.keys()):
            h.update(key.encode())
            h.update(f.get_tensor(key).float().numpy().tobytes())
    return h.hexdigest()


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_plain_matches_reference_logits(tmp_path, name):
    gold = np.load(GOLDEN / f"{name}.npz")
    cfg = json.loads(bytes(gold["config"]).decode())
    assert cfg == json.loads(json.dumps(H.CONFIGS[name][0], sort_keys=True))
    model_dir = H.make_model_dir(tmp_path, name)
    assert _checksum(model_dir) == bytes(gold["checksum"]).decode(), (
        "the random-weights writer no longer draws the weights the golden file was made with"
    )
    tokens = gold["tokens"].tolist()
    for dtype, tol in ((torch.float64, 2e-6), (torch.float32, 5e-6)):
        model = pl.read_model(model_dir, dtype)
        logits = pl.forward(model, tokens).numpy()
        err = np.abs(logits - gold["logits"]).max()
        assert err <= tol, f"{name} {dtype}: {err}"
    assert np.abs(gold["chunked_last"] - gold["logits"][-1]).max() < 1e-6
    m = pl.read_model(model_dir, torch.float32)
    freqs = pl.rope_freqs(m.head_dim, cfg["rope_theta"], cfg.get("rope_scaling"))
    assert np.array_equal(freqs.numpy(), gold["rope_freqs"])


def test_plain_parts_are_consistent():
    """Attention of the plain implementation against a direct double loop."""
    torch.manual_seed(0)
    t, hq, hkv, hd = 9, 4, 2, 8
    q, k, v = (torch.randn(t, h, hd, dtype=torch.float64) for h in (hq, hkv, hkv))
    out = pl.causal_attention(q, k, v, hd ** -0.5, window=4)
    for i in range(t):
        for h in range(hq):
            js = [j for j in range(t) if j <= i and j > i - 4]
            s = torch.tensor([float(q[i, h] @ k[j, h // 2]) * hd ** -0.5 for j in js], dtype=torch.float64)
            p = torch.softmax(s, 0)
            ref = sum(p[n] * v[j, h // 2] for n, j in enumerate(js))
            assert torch.allclose(out[i, h], ref, atol=1e-12)
    w = torch.randn(16, 5, dtype=torch.float64)
    pw = pl.permute_qk_rows(w, 2)
    assert torch.equal(pw[0], w[0]) and torch.equal(pw[1], w[4]) and torch.equal(pw[9], w[12])
