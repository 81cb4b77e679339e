"""Weights from safetensors, by tensor name.

The reference reads ``model-*-of-*.safetensors`` shards and renames tensors to
its own names (fastgen/utils/loading.py:255-293, 86-147).  Here tensors keep
their checkpoint names; the model says which names and shapes it needs
(:class:`~fastgen_b200.parts.base.WeightSpec`) and the loader checks the files
against that list *before* reading any data, reporting every missing tensor,
every unexpected tensor and every wrong shape in one error.

Kept dtypes: tensors stored in 16-bit floating point become bfloat16; a tensor
stored in 32-bit floating point stays float32; integer tables become int32.
(The float32 compute path upcasts what it needs when the parts bind.)
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Iterable, List, Sequence, Union

import torch
from safetensors import safe_open

from ..parts.base import WeightSpec


class WeightError(RuntimeError):
    """The checkpoint does not hold what the model needs."""


def checkpoint_files(model_dir: Union[str, Path]) -> List[Path]:
    """``model.safetensors``, or the shards named by the index / by pattern."""
    model_dir = Path(model_dir)
    single = model_dir / "model.safetensors"
    if single.is_file():
        return [single]
    index = model_dir / "model.safetensors.index.json"
    if index.is_file():
        with open(index) as f:
            names = sorted(set(json.load(f)["weight_map"].values()))
        return [model_dir / n for n in names]
    shards = sorted(model_dir.glob("model-*-of-*.safetensors"))
    if shards:
        return shards
    raise WeightError(f"no safetensors file found in {model_dir}")


def _kept_dtype(stored: torch.dtype, integer: bool) -> torch.dtype:
    if integer:
        return torch.int32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def load_weights(
    model_dir: Union[str, Path],
    specs: Sequence[WeightSpec],
    device,
    ignore: Iterable[str] = (),
) -> Dict[str, torch.Tensor]:
    """Load the tensors named by ``specs`` onto ``device``.

    ``ignore`` names tensors that may be present without being used (a tied
    model that also ships its output matrix).
    """
    files = checkpoint_files(model_dir)
    wanted = {s.name: s for s in specs}
    ignore = set(ignore)
    where: Dict[str, Path] = {}
    shapes: Dict[str, tuple] = {}
    for path in files:
        if not path.is_file():
            raise WeightError(f"checkpoint shard {path} is missing")
        with safe_open(str(path), framework="pt", device="cpu") as f:
            for key in f.keys():
                where[key] = path
                shapes[key] = tuple(f.get_slice(key).get_shape())

    missing = sorted(n for n in wanted if n not in where)
    unexpected = sorted(n for n in where if n not in wanted and n not in ignore)
    wrong = [
        f"{n}: expected {tuple(wanted[n].shape)}, found {shapes[n]}"
        for n in sorted(wanted)
        if n in shapes and tuple(wanted[n].shape) != shapes[n]
    ]
    if missing or unexpected or wrong:
        lines = [f"checkpoint in {model_dir} does not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
        raise WeightError("\n".join(lines))

    out: Dict[str, torch.Tensor] = {}
    by_file: Dict[Path, List[str]] = {}
    for name in wanted:
        by_file.setdefault(where[name], []).append(name)
    for path, names in by_file.items():
        with safe_open(str(path), framework="pt", device="cpu") as f:
            for name in names:
                t = f.get_tensor(name)
                spec = wanted[name]
                if spec.integer and t.is_floating_point():
                    raise WeightError(f"{name}: expected an integer table, found {t.dtype}")
                if not spec.integer and not t.is_floating_point():
                    raise WeightError(f"{name}: expected floating point, found {t.dtype}")
                out[name] = t.to(device=device, dtype=_kept_dtype(t.dtype, spec.integer))
    return out
