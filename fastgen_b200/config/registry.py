"""The one registry from an architecture's name to its description builder.

The reference matches ``config["architectures"]`` against literal lists
(fastgen/utils/loading.py:235-244); here the table is open so that another
architecture is one ``register_architecture`` call.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Callable, Dict, Mapping, Union

from .model_args import ConfigError, ModelArgs

ArchBuilder = Callable[[Mapping[str, Any]], ModelArgs]

_ARCHITECTURES: Dict[str, ArchBuilder] = {}


def register_architecture(name: str, builder: ArchBuilder) -> None:
    """Register ``builder(config_dict) -> ModelArgs`` under ``name``."""
    _ARCHITECTURES[name] = builder


def architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def model_args_from_config(config: Mapping[str, Any]) -> ModelArgs:
    """Turn a parsed ``config.json`` into a :class:`ModelArgs`."""
    archs = config.get("architectures")
    if not isinstance(archs, (list, tuple)) or len(archs) != 1:
        raise ConfigError(
            "config.json must name exactly one architecture under "
            f"'architectures', got {archs!r}"
        )
    name = archs[0]
    builder = _ARCHITECTURES.get(name)
    if builder is None:
        raise ConfigError(
            f"unsupported architecture {name!r}; registered: {', '.join(architectures())}"
        )
    return builder(config)


def read_config(model_dir: Union[str, Path]) -> Dict[str, Any]:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"file {path} not found")
    with open(path) as f:
        try:
            config = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path} is not valid JSON: {e}") from None
    if not isinstance(config, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return config


def load_model_args(model_dir: Union[str, Path]) -> ModelArgs:
    """Read ``model_dir/config.json`` and build the model description.  A ``vocab_size``
    of -1 stands for the size of the folder's tokenizer (fastgen/generate.py:153-154)."""
    config = read_config(model_dir)
    if config.get("vocab_size") == -1:
        path = Path(model_dir) / "tokenizer.json"
        if not path.is_file():
            raise ConfigError(
                f"config.json gives vocab_size -1 (the tokenizer's), but {path} does not exist"
            )
        from tokenizers import Tokenizer

        config = dict(config, vocab_size=Tokenizer.from_file(str(path)).get_vocab_size())
    return model_args_from_config(config)
