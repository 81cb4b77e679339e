"""Make the golden logits: the reference's own model code, run once on the CPU.

Run from the repository root:

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/fastgen-checkout

What runs is the reference's code: its config parsing and weight renaming and
permutation (fastgen/utils/loading.py), its ``Transformer`` (fastgen/model.py),
its ``prefill``/``_forward`` with its rope table (fastgen/forward.py) and its
three Triton kernels under the Triton interpreter (fastgen/kernels).  The only
substitution is ``fastgen.forward.attention``: the reference calls the
flash-attn library there, which has no CPU path, so a plain paged
causal-softmax written from the call's arguments (forward.py:176-258) stands in.
Attention is therefore anchored on the formula only; everything else on the
reference's code.

Outputs ``tests/golden/<name>.npz`` with the token ids, the float32 logits of
every position (one ``prefill`` per prefix) and a checksum of the weights.
"""

import hashlib
import json
import os
import sys
import tempfile
from pathlib import Path

os.environ.setdefault("TRITON_INTERPRET", "1")
os.environ.setdefault("FG_NO_CUDA_GRAPHS", "1")

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))

import helpers as H  # noqa: E402


def weights_checksum(model_dir) -> str:
    from safetensors import safe_open

    h = hashlib.sha256()
    with safe_open(str(Path(model_dir) / "model.safetensors"), framework="pt", device="cpu") as f:
        for key in sorted(f.keys()):
            h.update(key.encode())
            h.update(f.get_tensor(key).float().numpy().tobytes())
    return h.hexdigest()


def paged_attention_shim(query, key, value, seqinfo, block_tbl, page_size):
    """softmax(q k^T * hd^-0.5) v, causal and bottom-right aligned, keys taken
    from the paged cache through the block table (arguments of forward.py:176-258)."""
    out = torch.empty_like(query)
    n_heads, hd = query.shape[1], query.shape[2]
    n_kv = key.shape[1]
    group = n_heads // n_kv
    q_start = seqinfo.q_seqstart.tolist()
    k_len = seqinfo.k_seqlen.tolist()
    for b in range(len(k_len)):
        qs, qe = q_start[b], q_start[b + 1]
        n, t = k_len[b], qe - qs
        slots = [int(block_tbl[b, j // page_size]) * page_size + j % page_size for j in range(n)]
        k = key[slots]
        v = value[slots]
        for h in range(n_heads):
            s = (query[qs:qe, h] @ k[:, h // group].T) * hd ** -0.5
            i = torch.arange(t)[:, None]
            j = torch.arange(n)[None, :]
            s = s.masked_fill(j > (n - t + i), float("-inf"))
            out[qs:qe, h] = torch.softmax(s, dim=-1) @ v[:, h // group]
    return out


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    import fastgen.forward as fwd
    from fastgen.cache import RawCache
    from fastgen.model import Transformer
    from fastgen.utils.loading import HfLoader

    fwd.attention = paged_attention_shim
    for name, n_tokens in (("tiny_a", 24), ("tiny_b", 40)):
        cfg, seed = H.CONFIGS[name]
        with tempfile.TemporaryDirectory() as tmp:
            model_dir = H.make_model_dir(tmp, name)
            # the reference only reads shards named model-*-of-*.safetensors
            os.rename(model_dir / "model.safetensors", model_dir / "model-00001-of-00001.safetensors")
            loader = HfLoader(model_dir)
            args = loader.load_model_args()
            torch.set_default_dtype(torch.float32)
            model = Transformer(args).to_empty(device="cpu")
            loader.load(model, show_progress=False)
            model = model.float()
            os.rename(model_dir / "model-00001-of-00001.safetensors", model_dir / "model.safetensors")
            checksum = weights_checksum(model_dir)
        tokens = H.random_tokens(cfg["vocab_size"], n_tokens, 42)
        page = 8
        n_pages = -(-n_tokens // page)
        rows = []
        for t in range(1, n_tokens + 1):
            cache = RawCache.build(model, n_pages * page, device=torch.device("cpu"), dtype=torch.float32)
            tbl = torch.arange(n_pages, dtype=torch.int32)[None, :]
            logits = fwd.prefill(model, torch.tensor(tokens[:t], dtype=torch.int32), [(0, t)], tbl, page, cache)
            rows.append(logits[0].numpy())
        # and once more in two portions, through the reference's own (n0, n1) interface
        cache = RawCache.build(model, n_pages * page, device=torch.device("cpu"), dtype=torch.float32)
        cut = n_tokens // 3
        fwd.prefill(model, torch.tensor(tokens[:cut], dtype=torch.int32), [(0, cut)], tbl, page, cache)
        chunked = fwd.prefill(model, torch.tensor(tokens[cut:], dtype=torch.int32),
                              [(cut, n_tokens - cut)], tbl, page, cache)[0].numpy()
        np.savez_compressed(
            HERE / f"{name}.npz",
            tokens=np.asarray(tokens, dtype=np.int32),
            logits=np.stack(rows).astype(np.float32),
            chunked_last=chunked.astype(np.float32),
            rope_freqs=model.rope_freqs.numpy(),
            checksum=np.frombuffer(checksum.encode(), dtype=np.uint8),
            config=np.frombuffer(json.dumps(cfg, sort_keys=True).encode(), dtype=np.uint8),
        )
        print(name, "written; whole vs chunked last-row diff",
              float(np.abs(chunked - rows[-1]).max()))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py /path/to/fastgen-checkout")
    main(sys.argv[1])
