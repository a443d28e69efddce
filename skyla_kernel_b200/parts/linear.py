"""Matrix products of the parts: picks the kernel for a weight, a precision and a row count.

``y = x W^T`` with ``W`` stored ``[outputs, inputs]`` (skyla-ref/src/matrix.rs:38-58).
The plain 32-bit kernel takes every shape and dtype; the tensor-core and
bandwidth-bound bfloat16 kernels take the shapes they are written for and are
chosen here, never by the caller.
"""
from __future__ import annotations

import torch

from ..kernels import ops

STORE, ACCUMULATE, GATED = ops.STORE, ops.ACCUMULATE, ops.GATED


class Linear:
    kernel_modules = ("linear_plain",)

    def __init__(self, weight: torch.Tensor, rt, gated_group: int = 0):
        """``weight`` on the device; ``gated_group`` > 0 marks a fused gate/up matrix."""
        self.weight = weight
        self.rt = rt
        self.gated_group = gated_group
        self.n_in = weight.shape[1]
        self.n_out = weight.shape[0] // 2 if gated_group else weight.shape[0]

    def forward(self, x: torch.Tensor, y: torch.Tensor, mode: int = STORE) -> torch.Tensor:
        if self.gated_group:
            mode = GATED
        return ops.linear_plain(x, self.weight, y, mode, self.gated_group)

    def bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()
