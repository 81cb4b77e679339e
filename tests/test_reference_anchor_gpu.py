"""The plain implementation's attention against the reference's own, on the GPU.

On the CPU the reference's model code runs with one function replaced: its
``attention`` (fastgen/forward.py:176-258) is a flash-attn call without a CPU path, so the
golden logits of ``tests/golden`` pin every formula of ``plain_llama.py`` except the
attention's scale, its bottom-right causal alignment for ``t`` queries on ``n`` keys and its
grouping of heads.  Here the reference runs unmodified on the device, in bfloat16, through its
own ``prefill`` (fastgen/forward.py:518-573): a model folder is loaded by its ``HfLoader``,
prompts go in whole, in two portions (``(n0, n1)`` pairs) and two at a time, and the logits it
returns (the last position of every sequence) are held to the plain implementation's under the
bfloat16 rule of ``helpers.check_row``.

Needs the reference installed under ``baseline/_ref`` (``pip install --target``; it is not part
of the repository) and the flash-attn package the reference imports; skipped otherwise.
"""

import os
import sys
from pathlib import Path

import pytest
import torch

import helpers as H
from fastgen_b200.weights import write_random_model

pytestmark = pytest.mark.gpu

REF = Path(__file__).resolve().parent.parent / "baseline" / "_ref"

# head sizes 64 and 128 (flash-attn takes them); the reference computes the head size as
# hidden_size / heads and knows no window, so the configurations say neither
ANCHOR = {
    "hd64": dict(
        architectures=["LlamaForCausalLM"], hidden_size=256, intermediate_size=344, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-5, vocab_size=300,
        tie_word_embeddings=False, rope_theta=10000.0, max_position_embeddings=1024,
    ),
    "hd128": dict(
        architectures=["LlamaForCausalLM"], hidden_size=384, intermediate_size=264, num_hidden_layers=3,
        num_attention_heads=3, num_key_value_heads=1, rms_norm_eps=1e-6, vocab_size=270,
        tie_word_embeddings=True, rope_theta=500000.0,
        rope_scaling=dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                          original_max_position_embeddings=64, rope_type="llama3"),
        max_position_embeddings=1024,
    ),
}
PAGE = 256  # flash-attn's paged cache wants pages that are multiples of 256


def _reference():
    if not (REF / "fastgen").is_dir():
        pytest.skip("the reference is not installed under baseline/_ref")
    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    try:
        import fastgen.forward as fwd
        from fastgen.cache import RawCache
        from fastgen.model import Transformer
        from fastgen.utils.loading import HfLoader
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"the reference does not import here: {e!r}")
    return fwd, RawCache, Transformer, HfLoader


@pytest.mark.parametrize("name", list(ANCHOR))
def test_plain_attention_matches_the_reference_on_the_device(tmp_path, name):
    fwd, RawCache, Transformer, HfLoader = _reference()
    cfg = ANCHOR[name]
    model_dir = write_random_model(tmp_path / name, cfg, seed=31, dtype=torch.bfloat16, norm_jitter=0.1)
    dev = torch.device("cuda:0")
    # the reference only reads shards named model-*-of-*.safetensors
    os.rename(model_dir / "model.safetensors", model_dir / "model-00001-of-00001.safetensors")
    old_dtype = torch.get_default_dtype()
    try:
        torch.set_default_dtype(torch.bfloat16)  # as fastgen/generate.py:156 does
        loader = HfLoader(model_dir)
        model = Transformer(loader.load_model_args()).to_empty(device=dev)
        loader.load(model, show_progress=False)
    finally:
        torch.set_default_dtype(old_dtype)
        os.rename(model_dir / "model-00001-of-00001.safetensors", model_dir / "model.safetensors")

    vocab = cfg["vocab_size"]
    a = H.random_tokens(vocab, 300, 1)
    b = H.random_tokens(vocab, 77, 2)
    ref_a, ref_b = H.plain_logits(model_dir, a), H.plain_logits(model_dir, b)
    n_pages = 4

    def cache():
        return RawCache.build(model, n_pages * PAGE, device=dev, dtype=torch.bfloat16)

    def toks(t):
        return torch.tensor(t, dtype=torch.int32, device=dev)

    tbl = torch.tensor([[0, 1], [2, 3]], dtype=torch.int32, device=dev)
    # the reference makes its frequency table and index tensors on the default device; its own
    # tools set that to the GPU (fastgen/tools/chat.py:47-48)
    with torch.inference_mode(), torch.device(dev):
        # whole prompts of several lengths: scale, grouping of the heads, the causal mask
        for t in (1, 2, 63, 64, 65, 130, 300):
            logits = fwd.prefill(model, toks(a[:t]), [(0, t)], tbl[:1], PAGE, cache())
            H.check_row(logits[0].float().cpu().numpy(), ref_a[t - 1], torch.bfloat16, f"whole {t}")
        # two portions: t queries on n keys, bottom-right aligned; cut inside and at the end of a tile
        for cut in (1, 64, 100, 299):
            c = cache()
            fwd.prefill(model, toks(a[:cut]), [(0, cut)], tbl[:1], PAGE, c)
            logits = fwd.prefill(model, toks(a[cut:]), [(cut, 300 - cut)], tbl[:1], PAGE, c)
            H.check_row(logits[0].float().cpu().numpy(), ref_a[299], torch.bfloat16, f"cut {cut}")
        # two sequences in one call, one of them a portion on cached keys
        c = cache()
        fwd.prefill(model, toks(a[:150]), [(0, 150)], tbl[:1], PAGE, c)
        logits = fwd.prefill(model, toks(a[150:] + b), [(150, 150), (0, len(b))], tbl, PAGE, c)
        H.check_row(logits[0].float().cpu().numpy(), ref_a[299], torch.bfloat16, "batched a")
        H.check_row(logits[1].float().cpu().numpy(), ref_b[len(b) - 1], torch.bfloat16, "batched b")
        # a decoded token is the pair (n - 1, 1)
        c = cache()
        fwd.prefill(model, toks(a[:199]), [(0, 199)], tbl[:1], PAGE, c)
        logits = fwd.prefill(model, toks(a[199:200]), [(199, 1)], tbl[:1], PAGE, c)
        H.check_row(logits[0].float().cpu().numpy(), ref_a[199], torch.bfloat16, "single token")
