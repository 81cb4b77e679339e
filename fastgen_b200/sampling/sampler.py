"""Greedy, temperature and top-p sampling on the device.

Options and meanings follow fastgen/generate.py:887-896 and
fastgen/utils/sampling.py:6-31: with ``use_sampling`` the next token is drawn
from ``softmax(logits / temperature)`` restricted to the nucleus ``top_p``;
without it the next token is ``argmax(logits)``.  A row whose temperature is
zero is greedy.  Draws are keyed by (seed, request key, position), so they do
not depend on how requests are batched or preempted.
"""

from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch


class Sampler:
    def __init__(self, ops, vocab_size: int, max_rows: int, use_sampling: bool = True,
                 top_p: float = 1.0, seed: int = 777, logprobs: bool = False) -> None:
        if not 0.0 < top_p:
            raise ValueError(f"top_p must be positive, got {top_p}")
        self.ops = ops
        self.vocab_size = vocab_size
        self.use_sampling = use_sampling
        self.top_p = float(top_p)
        self.seed = int(seed)
        self.logprobs = logprobs
        self.max_rows = max_rows
        self._scratch = None

    def _scratch_for(self, rows: int) -> torch.Tensor:
        need = rows * self.vocab_size
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.empty(max(need, min(self.max_rows, 64) * self.vocab_size),
                                        dtype=torch.float32, device=self.ops.device)
        return self._scratch

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], keys: Sequence[int],
               positions: Sequence[int]) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """Sample one token per row of ``logits`` [rows, vocab].  Returns device
        tensors (int32 ``[rows + 1]``: the tokens, then the device status word as the
        step's kernels left it; logprobs float32 ``[rows]`` or ``None``).  The status
        word comes with the tokens so that the caller's one read of them also tells it
        whether a kernel recorded a fault (``csrc.ops.describe_status``)."""
        rows = logits.shape[0]
        dev = self.ops.device
        out = torch.empty(rows + 1, dtype=torch.int32, device=dev)
        lp = torch.empty(rows, dtype=torch.float32, device=dev) if self.logprobs else None
        if self.use_sampling and any(t > 0 for t in temperatures):
            temps = torch.tensor(list(temperatures), dtype=torch.float32).to(dev)
            kk = torch.tensor(list(keys), dtype=torch.int64).to(dev)
            pp = torch.tensor(list(positions), dtype=torch.int32).to(dev)
            self.ops.sample(logits, temps, self.top_p, self.seed, kk, pp, out, lp, self._scratch_for(rows),
                            with_status=True)
        else:
            self.ops.sample(logits, None, 1.0, self.seed, None, None, out, lp, None, with_status=True)
        return out, lp
