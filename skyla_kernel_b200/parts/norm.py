"""RMSNorm: ``y = (x * r) * w`` with ``r = 1/sqrt(mean(x^2) + eps)``, in 32-bit.

The weight is used as stored, not ``1 + w`` (skyla-ref/src/ops.rs:1-16;
skyla-shaders/shaders/rmsnorm.comp:22-51).  ``width`` and ``eps`` are parameters.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Part, register_norm


class RMSNorm(Part):
    graph_safe = True
    kernel_modules = ("norm",)

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def declare(cls, spec) -> Dict[str, TensorDecl]:
        return {spec.tensors["weight"]: TensorDecl((int(spec.params["width"]),), "norm")}

    def load(self, tensors) -> None:
        self.weight = self.rt.vector(tensors[self.spec.tensors["weight"]])

    def forward(self, ctx, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None):
        return ops.rmsnorm(x, self.weight, self.eps, out, rows)

    def rms_scale_form(self):
        """``(weight, eps)``: this norm is ``x * weight / sqrt(mean(x^2) + eps)``, one scalar per row times a
        fixed vector.  A matrix product may use that: the scalar commutes with the product, so whoever
        writes ``x`` last can leave ``x * weight`` and the rows' sums of squares for the product that
        follows the norm ("norm ahead").  A norm of another form does not define this method."""
        return self.weight, self.eps

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()


register_norm("rmsnorm", RMSNorm)
