"""Arrangements of a layer's parts.

A block class takes a :class:`~skyla_kernel_b200.config.LayerSpec`, reads from its ``parts`` the
names it wants (each from the registry it chooses) and runs them on the residual stream.  What the
model asks of a block: ``declare(layer_spec)``, ``load(tensors)``, ``forward(ctx, x, entry)``,
``parts()``, ``kernels_needed()``, ``weight_bytes()``, ``cache_need()`` and ``state_need()`` (what a
run of the layer keeps in the cache: ``None`` for a block without a mixer), and optionally
``first_norm`` (the norm that reads ``x`` first, for the block before it).

``prenorm_residual``: ``x += mixer(mixer_norm(x)); x += feed_forward(ffn_norm(x))``
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


class Block:
    """Base of the arrangements: builds the parts that ``PARTS`` names from the layer's spec and does
    the housekeeping; a subclass says which parts it wants and how a step runs through them."""

    #: (name in ``LayerSpec.parts``, registry it comes from) of every part, in the order they load
    PARTS = ()
    #: name of the part whose cache and state needs are the layer's (``None``: the layer keeps nothing)
    CACHING_PART = "mixer"

    def __init__(self, layer_spec, rt):
        self.spec = layer_spec
        self.rt = rt
        for name, category in self.PARTS:
            setattr(self, name, build_part(category, layer_spec.part(name), rt))

    def parts(self):
        return tuple(getattr(self, name) for name, _ in self.PARTS)

    @classmethod
    def declare(cls, layer_spec):
        d = {}
        for name, category in cls.PARTS:
            d.update(declare_part(category, layer_spec.part(name)))
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

    def cache_need(self):
        part = getattr(self, self.CACHING_PART, None) if self.CACHING_PART else None
        return part.cache_need() if part is not None else None

    def state_need(self):
        part = getattr(self, self.CACHING_PART, None) if self.CACHING_PART else None
        return part.state_need() if part is not None else None

    def forward(self, ctx, x, entry: EntryBinding) -> None:
        raise NotImplementedError


class PrenormResidualBlock(Block):
    PARTS = (("mixer_norm", "norm"), ("mixer", "mixer"), ("ffn_norm", "norm"), ("feed_forward", "feed_forward"))

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
