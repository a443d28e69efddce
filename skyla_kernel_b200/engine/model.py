"""A decoder assembled from a :class:`ModelSpec`: embedding, the scheduled runs
of its layers, final norm and head.

The forward pass follows skyla-ref/src/model.rs:97-122: embed, then for each
scheduled layer the block, then the final norm and the output product -- but for
a packed batch of new tokens, reading and writing the cache, and with the final
norm and the head applied only to the rows whose logits are wanted (the
reference norms and projects one row per replay, skyla-engine/src/graph.rs:219-230).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.base import ConfigError, ModelSpec
from ..kernels import build as kernel_build
from ..parts.base import Runtime, build_part, declare_part, part_class
from ..parts.block import EntryBinding
from ..weights.loader import TensorDecl


def declared_tensors(spec: ModelSpec) -> Dict[str, TensorDecl]:
    """Every tensor the model's parts will ask for, by checkpoint name."""
    d: Dict[str, TensorDecl] = {}

    def add(new: Dict[str, TensorDecl]):
        for name, decl in new.items():
            if name in d and tuple(d[name].shape) != tuple(decl.shape):
                raise ConfigError(f"tensor {name} is declared with shapes {d[name].shape} and {decl.shape}")
            d.setdefault(name, decl)

    add(declare_part("embedding", spec.embedding))
    for layer in spec.layers:
        add(part_class("block", layer.block).declare(layer))
    add(declare_part("norm", spec.final_norm))
    add(declare_part("head", spec.head))
    return d


class DecoderModel:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.embedding = build_part("embedding", spec.embedding, rt)
        self.blocks = [part_class("block", layer.block)(layer, rt) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, rt)
        self.head = build_part("head", spec.head, rt)
        # schedule -> cache entries: one per run that owns a cache
        self.entries: List[EntryBinding] = []
        self.kv_needs = []
        self.state_needs = []
        owner_entry: Dict[int, int] = {}
        for i, e in enumerate(spec.schedule):
            if not 0 <= e.layer < len(self.blocks):
                raise ConfigError(f"schedule entry {i} names layer {e.layer}, the model has {len(self.blocks)}")
            block = self.blocks[e.layer]
            if e.reads_cache_of is None:
                owner_entry[i] = len(self.kv_needs)
                self.entries.append(EntryBinding(len(self.kv_needs), True))
                self.kv_needs.append(block.cache_need())
                self.state_needs.append(block.state_need())
            else:
                j = e.reads_cache_of
                if j not in owner_entry or j >= i:
                    raise ConfigError(f"schedule entry {i} reads the cache of entry {j}, which is not "
                                      f"an earlier entry with a cache of its own")
                src = self.blocks[spec.schedule[j].layer]
                if src.cache_need() != block.cache_need():
                    raise ConfigError(f"schedule entry {i} cannot read the cache of entry {j}: "
                                      f"their mixers need different caches")
                self.entries.append(EntryBinding(owner_entry[j], False))

    def graph_safe(self) -> bool:
        """Whether every part only launches kernels on the current stream with device-side
        control, so that a decode step can be captured in a CUDA graph and replayed."""
        parts = [self.embedding, self.final_norm, self.head]
        for b in self.blocks:
            parts.extend(b.parts())
        return all(getattr(p, "graph_safe", False) for p in parts)

    def tile_heights(self):
        """The heights of token tiles that the mixers want listed in every step's batch."""
        hs = []
        for b in self.blocks:
            for p in b.parts():
                hs.extend(getattr(p, "token_tiles", ()))
        return tuple(sorted(set(hs)))

    def step_plans(self):
        """The host-made plans that the parts want in every step's batch, one per key."""
        plans = {}
        for b in self.blocks:
            for p in b.parts():
                for plan in getattr(p, "step_plans", ()):
                    plans.setdefault(plan.key, plan)
        return tuple(plans.values())

    def kernels_needed(self):
        mods = list(self.embedding.kernels_needed())
        for b in self.blocks:
            mods.extend(b.kernels_needed())
        mods.extend(self.final_norm.kernels_needed())
        mods.extend(self.head.kernels_needed())
        return tuple(dict.fromkeys(mods))

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.embedding.load(tensors)
        for b in self.blocks:
            b.load(tensors)
        self.final_norm.load(tensors)
        self.head.load(tensors)
        self.rt.forget_host_tensors()

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights a decode step has to read: every scheduled layer and the head once."""
        total = self.head.weight_bytes() + self.final_norm.weight_bytes()
        for e in self.spec.schedule:
            total += self.blocks[e.layer].weight_bytes()
        return total

    def forward(self, ctx, taps: Optional[Dict[int, torch.Tensor]] = None) -> torch.Tensor:
        """Runs the step's tokens; returns float32 logits ``[wanted, vocab]``.

        ``taps``: schedule index -> tensor that receives the residual stream after
        that run (the reference's layer taps, skyla-engine/src/taps.rs:7-46).
        """
        hidden = self.spec.hidden_size
        x = ctx.buffer("model.x", (ctx.n_tokens, hidden), torch.float32)
        self.embedding.forward(ctx, ctx.tokens, x)
        ctx.mark("embedding")
        schedule = self.spec.schedule
        for i, e in enumerate(schedule):
            # the norm that reads x after this run, for a product that can prepare its input
            nxt = self.blocks[schedule[i + 1].layer] if i + 1 < len(schedule) else None
            ctx.after_block_norm = getattr(nxt, "first_norm", None)
            self.blocks[e.layer].forward(ctx, x, self.entries[i])
            if taps is not None and i in taps:
                taps[i].copy_(x)
        logits = ctx.buffer("model.logits", (ctx.n_want, self.spec.vocab_size), torch.float32)
        if ctx.n_want:
            h = ctx.buffer("model.final", (ctx.n_want, hidden), self.rt.act_dtype)
            self.final_norm.forward(ctx, x, h, rows=ctx.want)
            ctx.mark("take wanted rows + rmsnorm")
            self.head.forward(ctx, h, logits)
            ctx.mark("matvec output")
        ctx.ahead = ctx.next_norm = ctx.after_block_norm = None
        return logits
