"""Arrangements of a layer's parts.

``prenorm_residual``: ``x += mixer(norm_a(x)); x += feed_forward(norm_b(x))``
(skyla-ref/src/model.rs:104-115).  The residual stream ``x`` is 32-bit in every
precision; the mixer and the feed-forward add into it themselves, in the epilogue
of their last matrix product.
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import NormedInput, build_part, declare_part, register_block


@dataclass
class EntryBinding:
    """How one run of a layer is tied to the cache.

    ``cache_entry`` indexes the cache's entries (keys/values and state);
    ``owns_cache`` is false for a run that reads the entry another run wrote.
    """

    cache_entry: int
    owns_cache: bool = True


class PrenormResidualBlock:
    def __init__(self, layer_spec, rt):
        self.spec = layer_spec
        self.rt = rt
        self.mixer_norm = build_part("norm", layer_spec.mixer_norm, rt)
        self.mixer = build_part("mixer", layer_spec.mixer, rt)
        self.ffn_norm = build_part("norm", layer_spec.ffn_norm, rt)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, rt)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)

    @classmethod
    def declare(cls, layer_spec):
        d = {}
        for cat, spec in (("norm", layer_spec.mixer_norm), ("mixer", layer_spec.mixer),
                          ("norm", layer_spec.ffn_norm), ("feed_forward", layer_spec.feed_forward)):
            d.update(declare_part(cat, spec))
        return d

    def load(self, tensors) -> None:
        for p in self.parts():
            p.load(tensors)

    def kernels_needed(self):
        mods = []
        for p in self.parts():
            mods.extend(p.kernels_needed())
        return tuple(dict.fromkeys(mods))

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.parts())

    @property
    def first_norm(self):
        """The norm that reads the residual stream first when this block runs."""
        return self.mixer_norm

    def forward(self, ctx, x, entry: EntryBinding) -> None:
        after = getattr(ctx, "after_block_norm", None)
        h = NormedInput(ctx, x, self.mixer_norm)
        ctx.next_norm = self.ffn_norm  # who reads x after the mixer has added to it
        self.mixer.forward(ctx, h if getattr(self.mixer, "takes_normed_input", False) else h.tensor(), x, entry)
        h = NormedInput(ctx, x, self.ffn_norm)
        ctx.next_norm = after          # who reads x after the feed-forward has added to it
        self.feed_forward.forward(ctx, h if getattr(self.feed_forward, "takes_normed_input", False) else h.tensor(), x)
        ctx.next_norm = None


register_block("prenorm_residual", PrenormResidualBlock)
