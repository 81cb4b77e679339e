from .model_args import (
    ConfigError,
    LayerSpec,
    ModelArgs,
    PartSpec,
    ScheduleEntry,
)
from .registry import (
    architectures,
    load_model_args,
    model_args_from_config,
    read_config,
    register_architecture,
)
from . import llama as _llama  # registers LlamaForCausalLM

__all__ = [
    "ConfigError",
    "LayerSpec",
    "ModelArgs",
    "PartSpec",
    "ScheduleEntry",
    "architectures",
    "load_model_args",
    "model_args_from_config",
    "read_config",
    "register_architecture",
]
