"""Configuration, registry and weight loading (no GPU)."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

import helpers as H
import plain_llama as pl
from fastgen_b200.config import ConfigError, load_model_args, model_args_from_config, register_architecture
from fastgen_b200.engine.model import model_weight_specs
from fastgen_b200.parts.position import rope_frequencies
from fastgen_b200.weights import WeightError, load_weights, write_random_model


def test_llama_args_follow_config():
    for name, (cfg, _) in H.CONFIGS.items():
        args = model_args_from_config(cfg)
        assert args.dim == cfg["hidden_size"] and args.vocab_size == cfg["vocab_size"]
        assert len(args.layers) == cfg["num_hidden_layers"] == len(args.schedule)
        att = args.layers[0].mixer.params
        assert att.n_heads == cfg["num_attention_heads"]
        assert att.n_kv_heads == cfg["num_key_value_heads"]
        assert att.head_dim == cfg.get("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
        assert att.window == cfg.get("sliding_window")
        assert args.layers[0].ffn.params.ffn_dim == cfg["intermediate_size"]
        assert args.layers[0].mixer_norm.params.eps == cfg["rms_norm_eps"]
        assert args.tie_embeddings == cfg["tie_word_embeddings"]
        assert args.max_positions == cfg["max_position_embeddings"]
        rope = att.position.params
        assert rope.theta == cfg["rope_theta"]
        assert (rope.scaling is not None) == ("rope_scaling" in cfg)


def test_kv_heads_default_to_heads():
    cfg = dict(H.TINY_A)
    del cfg["num_key_value_heads"]
    assert model_args_from_config(cfg).layers[0].mixer.params.n_kv_heads == 4


def test_missing_keys_are_all_named():
    cfg = dict(H.TINY_A)
    del cfg["rms_norm_eps"], cfg["rope_theta"]
    with pytest.raises(ConfigError) as e:
        model_args_from_config(cfg)
    assert "rms_norm_eps" in str(e.value) and "rope_theta" in str(e.value)


def test_unknown_architecture_and_bad_sizes():
    with pytest.raises(ConfigError, match="FooForCausalLM"):
        model_args_from_config(dict(H.TINY_A, architectures=["FooForCausalLM"]))
    with pytest.raises(ConfigError, match="head size"):
        model_args_from_config(dict(H.TINY_A, head_dim=24))
    with pytest.raises(ConfigError, match="grouped"):
        model_args_from_config(dict(H.TINY_A, num_key_value_heads=3))
    with pytest.raises(ConfigError, match="positive"):
        model_args_from_config(dict(H.TINY_A, hidden_size=0))


def test_missing_config_file(tmp_path):
    with pytest.raises(ConfigError, match="not found"):
        load_model_args(tmp_path)


def test_registry_is_open():
    register_architecture("EchoForCausalLM", lambda cfg: model_args_from_config(dict(cfg, architectures=["LlamaForCausalLM"])))
    args = model_args_from_config(dict(H.TINY_A, architectures=["EchoForCausalLM"]))
    assert args.dim == 64


def test_rope_table_matches_plain():
    for name, (cfg, _) in H.CONFIGS.items():
        args = model_args_from_config(cfg)
        ours = rope_frequencies(args.layers[0].mixer.params.position.params)
        hd = args.layers[0].mixer.params.head_dim
        ref = pl.rope_freqs(hd, cfg["rope_theta"], cfg.get("rope_scaling"))
        assert torch.equal(ours, ref), name
    # the 8B table crosses all three branches of the scaling law
    big = dict(H.TINY_B, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
               rope_scaling=dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                 original_max_position_embeddings=8192))
    args = model_args_from_config(big)
    ours = rope_frequencies(args.layers[0].mixer.params.position.params)
    ref = pl.rope_freqs(128, 500000.0, big["rope_scaling"])
    assert torch.equal(ours, ref)


def test_random_model_folder_round_trip(tmp_path):
    d = H.make_model_dir(tmp_path, "tiny_b")
    cfg = json.load(open(d / "config.json"))
    assert cfg == H.TINY_B
    args = load_model_args(d)
    specs = model_weight_specs(args)
    tensors = load_weights(d, specs, "cpu")
    assert set(tensors) == {s.name for s in specs}
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    n_params = sum(t.numel() for t in tensors.values())
    assert n_params == 1_340_736
    # same seed, same weights; another seed, other weights
    d2 = write_random_model(tmp_path / "again", H.TINY_B, 2, norm_jitter=0.1)
    d3 = write_random_model(tmp_path / "other", H.TINY_B, 3, norm_jitter=0.1)
    a, b, c = (load_file(str(x / "model.safetensors")) for x in (d, d2, d3))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["lm_head.weight"], c["lm_head.weight"])
    norm = a["model.norm.weight"].float()
    assert 0.89 < norm.min() and norm.max() < 1.11 and norm.std() > 0.01


def test_tied_model_has_no_output_tensor(tmp_path):
    d = H.make_model_dir(tmp_path, "tiny_a")
    names = set(load_file(str(d / "model.safetensors")))
    assert "lm_head.weight" not in names and "model.embed_tokens.weight" in names
    assert sum(t.numel() for t in load_file(str(d / "model.safetensors")).values()) == 104_768


def test_weight_errors_list_everything(tmp_path):
    d = H.make_model_dir(tmp_path, "tiny_a")
    tensors = load_file(str(d / "model.safetensors"))
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.extra.weight"] = torch.zeros(3)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(32, 64, dtype=torch.bfloat16)
    save_file(tensors, str(d / "model.safetensors"))
    specs = model_weight_specs(load_model_args(d))
    with pytest.raises(WeightError) as e:
        load_weights(d, specs, "cpu")
    msg = str(e.value)
    assert "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "model.layers.0.extra.weight" in msg
    assert "model.layers.0.self_attn.k_proj.weight: expected (16, 64), found (32, 64)" in msg


def test_kept_dtypes(tmp_path):
    d = H.make_model_dir(tmp_path, "tiny_a")
    tensors = load_file(str(d / "model.safetensors"))
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()
    tensors["model.layers.0.mlp.up_proj.weight"] = tensors["model.layers.0.mlp.up_proj.weight"].half()
    save_file(tensors, str(d / "model.safetensors"))
    out = load_weights(d, model_weight_specs(load_model_args(d)), "cpu")
    assert out["model.norm.weight"].dtype == torch.float32  # stored in 32-bit, stays so
    assert out["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16
    assert out["model.embed_tokens.weight"].dtype == torch.bfloat16


def test_no_checkpoint(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(H.TINY_A))
    with pytest.raises(WeightError, match="no safetensors"):
        load_weights(tmp_path, [], "cpu")


def test_sharded_checkpoint(tmp_path):
    d = H.make_model_dir(tmp_path, "tiny_a")
    tensors = load_file(str(d / "model.safetensors"))
    keys = sorted(tensors)
    half = len(keys) // 2
    save_file({k: tensors[k] for k in keys[:half]}, str(d / "model-00001-of-00002.safetensors"))
    save_file({k: tensors[k] for k in keys[half:]}, str(d / "model-00002-of-00002.safetensors"))
    (d / "model.safetensors").unlink()
    out = load_weights(d, model_weight_specs(load_model_args(d)), "cpu")
    assert all(torch.equal(out[k], tensors[k]) for k in keys)
