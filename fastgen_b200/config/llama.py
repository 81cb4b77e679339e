"""``LlamaForCausalLM``: config.json keys -> model description.

Keys and defaults follow fastgen/utils/loading.py:53-84; tensor names follow
fastgen/utils/loading.py:86-147 (kept as the checkpoint spells them).
"""

from __future__ import annotations

from typing import Any, Mapping

from ..parts.params import (
    AttentionParams,
    Llama3Scaling,
    RMSNormParams,
    RopeParams,
    SwiGLUParams,
)
from .model_args import (
    ConfigError,
    LayerSpec,
    ModelArgs,
    PartSpec,
    ScheduleEntry,
    positive_int,
    require,
)
from .registry import register_architecture

_REQUIRED = (
    "hidden_size",
    "intermediate_size",
    "num_hidden_layers",
    "num_attention_heads",
    "rms_norm_eps",
    "vocab_size",
    "tie_word_embeddings",
    "rope_theta",
    "max_position_embeddings",
)

_SCALING_REQUIRED = (
    "factor",
    "low_freq_factor",
    "high_freq_factor",
    "original_max_position_embeddings",
)


def _stop_tokens(config: Mapping[str, Any]) -> tuple[int, ...]:
    eos = config.get("eos_token_id")
    if eos is None:
        return ()
    if isinstance(eos, int):
        return (eos,)
    return tuple(int(t) for t in eos)


def llama_model_args(config: Mapping[str, Any]) -> ModelArgs:
    require(config, _REQUIRED, "LlamaForCausalLM config.json")
    dim = positive_int(config, "hidden_size")
    n_heads = positive_int(config, "num_attention_heads")
    n_kv_heads = (
        positive_int(config, "num_key_value_heads")
        if config.get("num_key_value_heads") is not None
        else n_heads
    )
    if config.get("head_dim") is not None:
        head_dim = positive_int(config, "head_dim")
    else:
        if dim % n_heads != 0:
            raise ConfigError(
                f"hidden_size {dim} is not a multiple of num_attention_heads {n_heads}"
            )
        head_dim = dim // n_heads
    eps = float(config["rms_norm_eps"])
    n_layers = positive_int(config, "num_hidden_layers")
    ffn_dim = positive_int(config, "intermediate_size")

    scaling = None
    # Any truthy rope_scaling dict is read as the llama3 law (loading.py:75-82).
    if scaling_config := config.get("rope_scaling"):
        require(scaling_config, _SCALING_REQUIRED, "rope_scaling")
        scaling = Llama3Scaling(
            factor=float(scaling_config["factor"]),
            low_freq_factor=float(scaling_config["low_freq_factor"]),
            high_freq_factor=float(scaling_config["high_freq_factor"]),
            original_max_positions=int(
                scaling_config["original_max_position_embeddings"]
            ),
        )
    rope = PartSpec(
        "rope",
        RopeParams(head_dim=head_dim, theta=float(config["rope_theta"]), scaling=scaling),
    )
    window = config.get("sliding_window")
    if window is not None:
        window = positive_int(config, "sliding_window")

    try:
        attention = AttentionParams(
            dim=dim,
            n_heads=n_heads,
            n_kv_heads=n_kv_heads,
            head_dim=head_dim,
            position=rope,
            window=window,
            qk_layout="half_split",  # how Hugging Face Llama checkpoints store q_proj and k_proj
        )
    except ValueError as e:
        raise ConfigError(str(e)) from None

    layers = []
    for i in range(n_layers):
        p = f"model.layers.{i}."
        layers.append(
            LayerSpec(
                block="prenorm",
                mixer=PartSpec(
                    "gqa_attention",
                    attention,
                    {
                        "wq": p + "self_attn.q_proj.weight",
                        "wk": p + "self_attn.k_proj.weight",
                        "wv": p + "self_attn.v_proj.weight",
                        "wo": p + "self_attn.o_proj.weight",
                    },
                ),
                mixer_norm=PartSpec(
                    "rmsnorm",
                    RMSNormParams(dim, eps),
                    {"weight": p + "input_layernorm.weight"},
                ),
                ffn=PartSpec(
                    "swiglu",
                    SwiGLUParams(dim, ffn_dim),
                    {
                        "w1": p + "mlp.gate_proj.weight",
                        "w3": p + "mlp.up_proj.weight",
                        "w2": p + "mlp.down_proj.weight",
                    },
                ),
                ffn_norm=PartSpec(
                    "rmsnorm",
                    RMSNormParams(dim, eps),
                    {"weight": p + "post_attention_layernorm.weight"},
                ),
            )
        )
    tied = bool(config["tie_word_embeddings"])
    return ModelArgs(
        architecture="LlamaForCausalLM",
        dim=dim,
        vocab_size=positive_int(config, "vocab_size"),
        max_positions=positive_int(config, "max_position_embeddings"),
        tie_embeddings=tied,
        embedding_name="model.embed_tokens.weight",
        output_name=None if tied else "lm_head.weight",
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(n_layers)),
        final_norm=PartSpec(
            "rmsnorm", RMSNormParams(dim, eps), {"weight": "model.norm.weight"}
        ),
        stop_tokens=_stop_tokens(config),
    )


register_architecture("LlamaForCausalLM", llama_model_args)
