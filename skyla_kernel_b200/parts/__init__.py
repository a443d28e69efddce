"""Parts that layers are put together from, and their registries."""
from . import attention, block, embedding, feedforward, norm, rope  # noqa: F401  (registration)
from .base import (Part, Runtime, build_part, declare_part, part_class, register_block,
                   register_embedding, register_feed_forward, register_head, register_mixer,
                   register_norm, register_position)
from .base import NormedInput
from .block import Block, EntryBinding

__all__ = ["Part", "Runtime", "build_part", "declare_part", "part_class", "register_block",
           "register_embedding", "register_feed_forward", "register_head", "register_mixer",
           "register_norm", "register_position", "EntryBinding", "Block", "NormedInput"]
