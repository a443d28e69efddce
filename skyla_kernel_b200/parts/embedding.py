"""Token embedding and output head.

Embedding: ``x = E[token]``, no scaling (skyla-ref/src/model.rs:99-100).  Head:
``logits = W h`` in 32-bit; when the checkpoint has no output matrix the spec
names the embedding's tensor and both parts share one device copy
(skyla-ref/src/model.rs:70-73, skyla-engine/src/weights.rs:88-91).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Part, register_embedding, register_head
from .linear import STORE, Linear


class TokenEmbedding(Part):
    graph_safe = True
    kernel_modules = ("embed",)

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.weight = None

    @classmethod
    def declare(cls, spec) -> Dict[str, TensorDecl]:
        return {spec.tensors["weight"]: TensorDecl((int(spec.params["vocab_size"]),
                                                    int(spec.params["hidden_size"])))}

    def load(self, tensors) -> None:
        self.weight = self.rt.matrix(tensors[self.spec.tensors["weight"]], shared=True)

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, ctx, tokens: torch.Tensor, x: torch.Tensor) -> None:
        ops.embed_gather(tokens, self.weight, x, state=self.rt.kernel_state)


class LinearHead(Part):
    graph_safe = True
    kernel_modules = Linear.kernel_modules

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.proj: Linear = None

    @classmethod
    def declare(cls, spec) -> Dict[str, TensorDecl]:
        return {spec.tensors["weight"]: TensorDecl((int(spec.params["vocab_size"]),
                                                    int(spec.params["hidden_size"])))}

    def load(self, tensors) -> None:
        self.proj = Linear(self.rt.matrix(tensors[self.spec.tensors["weight"]], shared=True), self.rt)

    def weight_bytes(self) -> int:
        return self.proj.bytes()

    def forward(self, ctx, h: torch.Tensor, logits: torch.Tensor) -> None:
        self.proj.forward(h, logits, STORE)


register_embedding("token_embedding", TokenEmbedding)
register_head("linear_head", LinearHead)
