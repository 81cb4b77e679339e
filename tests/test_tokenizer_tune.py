"""The tokenizer wrapper, ``vocab_size = -1``, the memory budget and the q/k row layout (no GPU)."""

import json
import sys
from pathlib import Path

import pytest
import torch

import helpers as H
import plain_llama as pl
from fastgen_b200.config import ConfigError, load_model_args
from fastgen_b200.engine.tune import mem_params

REF = Path(__file__).resolve().parent.parent / "baseline" / "_ref"

WORDS = ["<s>", "</s>", "<unk>", "user", "assistant", ":", "hello", "world", "how", "are", "you", "\n"]
TEMPLATE = ("{{ bos_token }} {% for m in messages %}{{ m['role'] }} : {{ m['content'] }} \n {% endfor %}"
            "{% if add_generation_prompt %}assistant :{% endif %}")


def _tokenizer_folder(tmp_path, with_template=True) -> Path:
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import WhitespaceSplit

    d = Path(tmp_path) / "tok"
    d.mkdir()
    tk = Tokenizer(WordLevel({w: i for i, w in enumerate(WORDS)}, unk_token="<unk>"))
    tk.pre_tokenizer = WhitespaceSplit()
    tk.save(str(d / "tokenizer.json"))
    cfg = dict(bos_token="<s>", eos_token=dict(content="</s>"))
    if with_template:
        cfg["chat_template"] = TEMPLATE
    (d / "tokenizer_config.json").write_text(json.dumps(cfg))
    return d


def test_tokenizer_wrapper(tmp_path):
    """fastgen/utils/tokenizer.py:48-118: encode / decode, the chat template, stop tokens."""
    from fastgen_b200.utils.tokenizer import HfTokenizer

    tk = HfTokenizer(_tokenizer_folder(tmp_path))
    assert tk.vocab_size == len(WORDS)
    assert tk.encode("hello world") == [6, 7] and tk.decode([6, 7]) == "hello world"
    assert tk.id_to_str(1) == "</s>" and tk.str_to_id("you") == 10
    with pytest.raises(KeyError):
        tk.str_to_id("nope")
    assert tk.stop_tokens == [1]  # the eos token, given as a dict with "content"
    dialog = [dict(role="user", content="hello"), dict(role="assistant", content="world"),
              dict(role="user", content="how are you")]
    ids = tk.encode_dialog(dialog)
    words = [WORDS[i] for i in ids]
    assert words == ["<s>", "user", ":", "hello", "assistant", ":", "world", "user", ":", "how", "are", "you",
                     "assistant", ":"]
    assert [WORDS[i] for i in tk.encode_dialog(dialog, for_completion=False)] == words[:-2]


def test_tokenizer_errors(tmp_path):
    from fastgen_b200.utils.tokenizer import HfTokenizer

    with pytest.raises(RuntimeError, match="Could not find"):
        HfTokenizer(tmp_path)
    tk = HfTokenizer(_tokenizer_folder(tmp_path, with_template=False))
    with pytest.raises(RuntimeError, match="no chat template"):
        tk.encode_dialog([dict(role="user", content="hello")])


def test_vocab_size_minus_one_is_the_tokenizers(tmp_path):
    """fastgen/generate.py:153-154."""
    d = _tokenizer_folder(tmp_path)
    (d / "config.json").write_text(json.dumps(dict(H.TINY_A, vocab_size=-1)))
    assert load_model_args(d).vocab_size == len(WORDS)
    (d / "tokenizer.json").unlink()
    with pytest.raises(ConfigError, match="vocab_size -1"):
        load_model_args(d)
    (d / "config.json").write_text(json.dumps(dict(H.TINY_A, vocab_size=-2)))
    with pytest.raises(ConfigError, match="positive"):
        load_model_args(d)


def test_mem_params_formula():
    """fastgen/utils/tune.py:31-84 with the 8B sizes, by hand."""
    weights = 16_060_522_496
    mp = mem_params(weights, 131072, 4096, 14336, 2, 0.5, 40)
    assert mp.cache_tokens == (40_000_000_000 - weights - 500_000_000) // 131072
    assert mp.prefill_tokens == 500_000_000 // int((2 * 2 * 4096 + 2 * 2 * 14336) * 1.2)
    mp.round_to(256)
    assert mp.cache_tokens % 256 == 0 and mp.prefill_tokens % 256 == 0
    # a budget below the weights leaves no cache (tune.py:78: avail = max(prefill, ...))
    assert mem_params(weights, 131072, 4096, 14336, 2, 0.5, 10).cache_tokens == 0


@pytest.mark.parametrize("name", ["tiny_b", "tiny_d"])
def test_mem_params_equal_the_references(name):
    """The same numbers as the reference's own function on its own model object."""
    if not (REF / "fastgen").is_dir():
        pytest.skip("the reference is not installed under baseline/_ref")
    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    try:
        from fastgen.model import Transformer
        from fastgen.utils import tune as ref_tune
        from fastgen.utils.loading import LlamaForCausalLM
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"the reference does not import here: {e!r}")
    from fastgen_b200.config import model_args_from_config
    from fastgen_b200.engine.model import model_weight_specs

    cfg = H.CONFIGS[name][0]
    old = torch.get_default_dtype()
    try:
        torch.set_default_dtype(torch.bfloat16)  # the reference's estimate assumes 2-byte values
        ref_model = Transformer(LlamaForCausalLM.model_args(cfg))  # parameters on the meta device
    finally:
        torch.set_default_dtype(old)
    args = model_args_from_config(cfg)
    weight_bytes = sum(2 * int(torch.Size(s.shape).numel()) for s in model_weight_specs(args))
    att = args.layers[0].mixer.params
    per_token = 2 * len(args.schedule) * att.n_kv_heads * att.head_dim * 2
    for prefill_gb, gpu_gb in ((0.1, 0.2), (0.5, 20.0), (0.1, 0.0001)):
        ours = mem_params(weight_bytes, per_token, args.dim, args.layers[0].ffn.params.ffn_dim, 2, prefill_gb, gpu_gb)
        theirs = ref_tune.mem_params(ref_model, prefill_gb, gpu_gb)
        assert (ours.cache_tokens, ours.prefill_tokens) == (theirs.cache_tokens, theirs.prefill_tokens)


class _HostOps:
    """What ``bind`` needs of the kernel set, on the CPU."""
    act_dtype = torch.float32
    device = torch.device("cpu")


@pytest.mark.parametrize("layout", ["half_split", "adjacent"])
def test_qk_rows_are_reordered_only_for_half_split_checkpoints(layout):
    from fastgen_b200.config import PartSpec
    from fastgen_b200.parts import make_mixer
    from fastgen_b200.parts.params import AttentionParams, RopeParams

    dim, hq, hkv, hd = 24, 4, 2, 16
    spec = PartSpec("gqa_attention",
                    AttentionParams(dim, hq, hkv, hd, PartSpec("rope", RopeParams(hd, 10000.0)), qk_layout=layout),
                    {"wq": "q", "wk": "k", "wv": "v", "wo": "o"})
    g = torch.Generator().manual_seed(0)
    w = {k: torch.randn(n * hd, dim, generator=g) for k, n in (("wq", hq), ("wk", hkv), ("wv", hkv))}
    w["wo"] = torch.randn(dim, hq * hd, generator=g)
    mixer = make_mixer(spec)
    mixer.bind(w, _HostOps())
    wq, wk, wv = mixer.wqkv[: hq * hd], mixer.wqkv[hq * hd : (hq + hkv) * hd], mixer.wqkv[(hq + hkv) * hd :]
    if layout == "half_split":
        assert torch.equal(wq, pl.permute_qk_rows(w["wq"], hq)) and torch.equal(wk, pl.permute_qk_rows(w["wk"], hkv))
        assert not torch.equal(wq, w["wq"])
    else:
        assert torch.equal(wq, w["wq"]) and torch.equal(wk, w["wk"])
    assert torch.equal(wv, w["wv"])
    with pytest.raises(ValueError, match="qk_layout"):
        AttentionParams(dim, hq, hkv, hd, None, qk_layout="pairs")
