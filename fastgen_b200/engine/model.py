"""The model: parts put together as the description says, and its forward pass.

The reference's ``Transformer`` only holds weights and its forward is one
function written for one architecture (fastgen/model.py:151-202,
fastgen/forward.py:347-515).  Here the model is generic: it builds one block
per :class:`~fastgen_b200.config.LayerSpec` from the part registries and runs
the schedule; nothing in this file knows what a mixer or feed-forward does.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..config import ModelArgs, load_model_args
from ..parts.base import (
    Block,
    CacheSpec,
    StateSpec,
    WeightSpec,
    make_block,
    make_feed_forward,
    make_mixer,
    make_norm,
)
from ..weights.loader import load_weights


_MAKERS = {"mixer": make_mixer, "norm": make_norm, "feed_forward": make_feed_forward}


def _build_blocks(args: ModelArgs) -> List[Block]:
    blocks = []
    for layer in args.layers:
        extra = {}
        for name, role, spec in layer.extra:
            if role not in _MAKERS:
                raise ValueError(f"part {name!r} of a layer has role {role!r}; known: {sorted(_MAKERS)}")
            extra[name] = _MAKERS[role](spec)
        blocks.append(
            make_block(
                layer.block,
                make_mixer(layer.mixer),
                make_norm(layer.mixer_norm),
                make_feed_forward(layer.ffn),
                make_norm(layer.ffn_norm),
                **extra,
            )
        )
    return blocks


def _embedding_specs(args: ModelArgs) -> List[WeightSpec]:
    specs = [WeightSpec(args.embedding_name, (args.vocab_size, args.dim))]
    if not args.tie_embeddings:
        specs.append(WeightSpec(args.output_name, (args.vocab_size, args.dim)))
    return specs


def _collect_specs(args: ModelArgs, blocks: Sequence[Block], final_norm) -> List[WeightSpec]:
    specs: Dict[str, WeightSpec] = {}
    ordered = [_embedding_specs(args)[0]]
    for block in blocks:
        for part in block.parts():
            ordered.extend(part.weight_specs())
    ordered.extend(final_norm.weight_specs())
    ordered.extend(_embedding_specs(args)[1:])
    for s in ordered:
        if s.name in specs and specs[s.name].shape != s.shape:
            raise ValueError(f"tensor {s.name} is asked for with two shapes")
        specs.setdefault(s.name, s)
    return list(specs.values())


def model_weight_specs(args: ModelArgs) -> List[WeightSpec]:
    """Every checkpoint tensor a model of this description needs, in a fixed order."""
    return _collect_specs(args, _build_blocks(args), make_norm(args.final_norm))


class Model:
    """Blocks, embedding and output of one model on one device."""

    def __init__(self, args: ModelArgs, ops) -> None:
        self.args = args
        self.ops = ops
        self.blocks = _build_blocks(args)
        self.final_norm = make_norm(args.final_norm)
        self.embedding: Optional[torch.Tensor] = None
        self.output: Optional[torch.Tensor] = None

    # -- description -----------------------------------------------------------
    def weight_specs(self) -> List[WeightSpec]:
        return _collect_specs(self.args, self.blocks, self.final_norm)

    def cache_specs(self) -> List[Optional[CacheSpec]]:
        return [self.blocks[e.layer].mixer.cache_spec() for e in self.args.schedule]

    def state_specs(self) -> List[Optional[StateSpec]]:
        return [self.blocks[e.layer].mixer.state_spec() for e in self.args.schedule]

    def kv_from(self) -> List[Optional[int]]:
        return [e.kv_from for e in self.args.schedule]

    def cache_bytes_per_token(self, elt_size: int) -> int:
        """Bytes of keys and values one token adds over all runs that own a cache."""
        total = 0
        for spec, src in zip(self.cache_specs(), self.kv_from()):
            if spec is not None and src is None:
                total += spec.n_pools * spec.n_kv_heads * spec.head_dim * elt_size
        return total

    def weight_bytes(self) -> int:
        """Bytes of every tensor a step reads (fused buffers, embedding once if tied)."""
        seen, total = set(), 0
        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        add(self.output)
        for block in self.blocks:
            for part in block.parts():
                for v in vars(part).values():
                    if isinstance(v, torch.Tensor):
                        add(v)
        for v in vars(self.final_norm).values():
            if isinstance(v, torch.Tensor):
                add(v)
        return total

    # -- weights -----------------------------------------------------------------
    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        dt = self.ops.act_dtype
        self.embedding = tensors[self.args.embedding_name].to(dt).contiguous()
        if self.args.tie_embeddings:
            self.output = self.embedding
        else:
            self.output = tensors[self.args.output_name].to(dt).contiguous()
        for block in self.blocks:
            for part in block.parts():
                part.bind({local: tensors[name] for local, name in part.names.items()}, self.ops)
        self.final_norm.bind(
            {local: tensors[name] for local, name in self.final_norm.names.items()}, self.ops
        )

    @staticmethod
    def load(model_dir, dtype: torch.dtype, device) -> "Model":
        """Read ``config.json`` and the safetensors of ``model_dir``."""
        from ..csrc.ops import Ops

        args = load_model_args(model_dir)
        model = Model(args, Ops(dtype, device))
        ignore = [args.output_name or "lm_head.weight"] if args.tie_embeddings else []
        tensors = load_weights(model_dir, model.weight_specs(), device, ignore=ignore)
        model.bind(tensors)
        del tensors
        return model

    @staticmethod
    def random(args: ModelArgs, dtype: torch.dtype, device, seed: int = 0) -> "Model":
        """A model with seeded random weights drawn on the device (no files):
        matrices N(0, 0.02), norm weights 1, as the random-weights writer does."""
        from ..csrc.ops import Ops

        model = Model(args, Ops(dtype, device))
        gen = torch.Generator(device=device).manual_seed(int(seed))
        tensors = {}
        for spec in model.weight_specs():
            if spec.init[0] == "normal":
                t = torch.empty(spec.shape, dtype=torch.bfloat16, device=device)
                t.normal_(0.0, spec.init[1], generator=gen)
            elif spec.init[0] == "ones":
                t = torch.ones(spec.shape, dtype=torch.bfloat16, device=device)
            else:
                t = torch.randint(0, spec.init[1], spec.shape, generator=gen, device=device, dtype=torch.int32)
            tensors[spec.name] = t
        model.bind(tensors)
        return model

    # -- forward -----------------------------------------------------------------
    def forward(self, ctx, memories) -> Optional[torch.Tensor]:
        """Run the step's tokens through the schedule.  Returns float32 logits
        ``[len(ctx.want_rows), vocab]`` (``None`` when no logits are wanted)."""
        ops = self.ops
        t = ctx.n_tokens
        h = torch.empty((t, self.args.dim), dtype=torch.float32, device=ops.device)
        ops.embedding(self.embedding, ctx.tokens, h)
        pending = None
        for e, entry in enumerate(self.args.schedule):
            h, pending = self.blocks[entry.layer].forward(h, pending, ctx, memories[e])
        if ctx.n_want == 0:
            return None
        if pending is None:
            x = self.final_norm.forward(h, rows=ctx.want_rows)
        else:
            x = self.final_norm.add_forward(h, pending, rows=ctx.want_rows)
        return ops.linear(x, self.output, out_dtype=torch.float32)
