"""Random-weights mode: write a model folder from a configuration and a seed.

The reference has no such mode (its parameters are ``to_empty``,
fastgen/generate.py:158).  The folder holds ``config.json`` and
``model.safetensors`` with exactly the tensors the model description asks for,
drawn tensor by tensor, in the order the model lists them, from one seeded CPU
generator in float32 and then rounded to the storage dtype.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping, Union

import torch
from safetensors.torch import save_file

from ..config import model_args_from_config
from ..parts.base import WeightSpec


def draw(spec: WeightSpec, gen: torch.Generator, norm_jitter: float = 0.0) -> torch.Tensor:
    kind = spec.init[0]
    if kind == "normal":
        return torch.randn(spec.shape, generator=gen, dtype=torch.float32) * spec.init[1]
    if kind == "ones":
        if norm_jitter:
            u = torch.rand(spec.shape, generator=gen, dtype=torch.float32)
            return 1.0 + (2.0 * u - 1.0) * norm_jitter
        return torch.ones(spec.shape, dtype=torch.float32)
    if kind == "randint":
        return torch.randint(0, spec.init[1], spec.shape, generator=gen, dtype=torch.int32)
    raise ValueError(f"unknown init law {spec.init!r} for {spec.name}")


def write_random_model(
    model_dir: Union[str, Path],
    config: Mapping[str, Any],
    seed: int,
    dtype: torch.dtype = torch.bfloat16,
    norm_jitter: float = 0.0,
    std: float = None,
) -> Path:
    """Write ``config.json`` and ``model.safetensors`` into ``model_dir``.

    Matrices and embeddings are N(0, 0.02) (or ``std``), norm weights 1, or
    ``1 + U(-norm_jitter, norm_jitter)`` when a jitter is given.
    """
    from ..engine.model import model_weight_specs  # late: avoids an import cycle

    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    args = model_args_from_config(config)
    gen = torch.Generator(device="cpu").manual_seed(int(seed))
    tensors = {}
    for spec in model_weight_specs(args):
        if std is not None and spec.init[0] == "normal":
            spec = WeightSpec(spec.name, spec.shape, ("normal", std), spec.integer)
        t = draw(spec, gen, norm_jitter)
        tensors[spec.name] = t if spec.integer else t.to(dtype)
    save_file(tensors, str(model_dir / "model.safetensors"))
    with open(model_dir / "config.json", "w") as f:
        json.dump(dict(config), f, indent=1)
    return model_dir
