"""Choosing the next token from 32-bit logits, on the device.

Greedy is an argmax (skyla-ref/src/ops.rs:36-41); the reference's chat mode
samples with temperature, top-k and top-p, defaults 0.6 / 40 / 0.95
(docs/roadmap.md:282-283).  A draw is keyed by ``(seed, request id, step)``, so a
request's tokens do not depend on the batch it is in.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from ..kernels import ops


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0   # 0: greedy
    top_k: int = 0             # 0: off
    top_p: float = 1.0         # 1: off
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")
        if self.top_k < 0:
            raise ValueError("top_k must not be negative")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0


CHAT_DEFAULTS = SamplingParams(temperature=0.6, top_k=40, top_p=0.95)


class Sampler:
    kernel_modules = ("sampling",)

    def __init__(self, params: SamplingParams, device, state: Optional["ops.KernelState"] = None):
        """``state``: the kernel state whose error word is raised when a row of logits offers no token
        (every logit NaN); the engine's own when an engine samples."""
        self.params = params
        self.device = torch.device(device)
        self.state = state

    def __call__(self, logits: torch.Tensor, req_ids: Sequence[int], steps: Sequence[int]) -> torch.Tensor:
        """int32 tokens ``[rows]`` on the device."""
        n = logits.shape[0]
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        p = self.params
        if p.greedy:
            return ops.sample(logits, out, state=self.state)
        keys = torch.tensor([list(req_ids), list(steps)], dtype=torch.int32).to(self.device)
        return ops.sample(logits, out, p.temperature, p.top_k, p.top_p, p.seed, keys[0].contiguous(),
                          keys[1].contiguous(), state=self.state)
