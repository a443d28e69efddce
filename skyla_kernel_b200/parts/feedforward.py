"""Dense gated feed-forward: ``x += Wdown( silu(Wgate h) * (Wup h) )``.

``silu(z) = z / (1 + exp(-z))`` (skyla-ref/src/ffn.rs:21-28, ops.rs:28-30); no
bias.  Gate and up are stored as one matrix so that one product computes both and
its epilogue multiplies them; the down product adds into the residual stream
(skyla-engine/src/graph.rs:174-184 does the same in four dispatches).
Parameters: ``hidden_size``, ``intermediate_size``.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..weights.loader import TensorDecl
from ..kernels import ops
from .base import NormedInput, Part, register_feed_forward
from .linear import ACCUMULATE, GATED, Linear


def fuse_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """One matrix: all gate rows, then the up rows of the same outputs."""
    return torch.cat((gate, up), dim=0).contiguous()


class SwiGLU(Part):
    graph_safe = True
    takes_normed_input = True
    kernel_modules = Linear.kernel_modules

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.gate_up: Linear = None
        self.down: Linear = None

    @classmethod
    def declare(cls, spec) -> Dict[str, TensorDecl]:
        h, i = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        t = spec.tensors
        return {t["gate_proj"]: TensorDecl((i, h)), t["up_proj"]: TensorDecl((i, h)),
                t["down_proj"]: TensorDecl((h, i))}

    def load(self, tensors) -> None:
        t = self.spec.tensors
        gate, up = tensors.pop(t["gate_proj"]), tensors.pop(t["up_proj"])  # taken out: they live on fused
        if gate.dtype != up.dtype:
            gate, up = gate.to(torch.float32), up.to(torch.float32)
        fused = fuse_gate_up(gate, up)
        del gate, up
        self.gate_up = Linear(self.rt.matrix(fused), self.rt, gated=True)
        self.down = Linear(self.rt.matrix(tensors[t["down_proj"]]), self.rt)

    def weight_bytes(self) -> int:
        return self.gate_up.bytes() + self.down.bytes()

    def forward(self, ctx, h, x: torch.Tensor) -> None:
        act = ctx.buffer("ffn.act", (ctx.n_tokens, self.inter), self.rt.act_dtype)
        scale_in = None
        if isinstance(h, NormedInput):
            if (h.ahead is not None and self.gate_up.takes_scale_in(ctx.n_tokens)
                    and ops.tc_linear_ok(h.ahead[0], self.gate_up.weight)):
                scale_in = (h.ahead[1], h.norm.rms_scale_form()[1])  # the product that wrote x last left x * norm weight
                h = h.ahead[0]
            else:
                h = h.tensor()
        self.gate_up.forward(h, act, GATED, scale_in=scale_in)
        ctx.mark("matvec gate+up, silu")
        self.down.forward(act, x, ACCUMULATE, ctx=ctx)
        ctx.mark("matvec down")


register_feed_forward("swiglu", SwiGLU)
