"""Architecture description as data.

A model is described by three things, none of which is code:

* a list of :class:`LayerSpec` -- for every layer which norm, mixer and
  feed-forward part it is made of, each with its own sizes and constants;
* a *schedule* -- the order in which layers run (:class:`ScheduleEntry`), which
  may name a layer twice or let an entry read the cache that another entry wrote;
* the model-level pieces: embedding, final norm and output head.

The reference makes room for this with a per-layer ``Mixer`` enum chosen by
``Config::recurrent(layer)`` (skyla-ref/src/model.rs:17-20,29-50,
skyla-ref/src/lib.rs:120-124) and an ``Ffn`` enum (skyla-ref/src/ffn.rs:6-19).
Here the choice is a string key into the part registries plus a parameter dict,
so a layer can be assembled without the part knowing which model it is in.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """A config.json that cannot describe a model of the architecture it names."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer.

    ``kind`` is a registry key, ``params`` the part's sizes and constants, and
    ``tensors`` maps the part's own names for its weights (``"q_proj"``) to the
    names they have in the checkpoint (``"model.layers.3.self_attn.q_proj.weight"``),
    so a part never builds a checkpoint name itself.
    """

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    tensors: Dict[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: its weight-name prefix, the arrangement of its parts and the parts themselves.

    ``block`` names the arrangement (a registry key) and ``parts`` the parts by the names that this
    arrangement gives them.  For the Qwen3 decoder the arrangement is ``"prenorm_residual"``,
    ``x += mixer(mixer_norm(x)); x += feed_forward(ffn_norm(x))`` (skyla-ref/src/model.rs:104-115),
    with the four parts ``mixer_norm, mixer, ffn_norm, feed_forward``.  Which names an arrangement
    wants, and to which registry each belongs, is the block class's business: one with a norm after
    each sub-layer too, or without a feed-forward, asks for other names and needs no change here.
    """

    prefix: str
    block: str
    parts: Dict[str, PartSpec]

    def part(self, name: str) -> PartSpec:
        try:
            return self.parts[name]
        except KeyError:
            have = ", ".join(sorted(self.parts)) or "(none)"
            raise ConfigError(f"layer {self.prefix!r}: the {self.block!r} block needs a part named {name!r}; "
                              f"the layer has {have}") from None


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer inside a step.

    ``layer`` indexes the layer list.  ``reads_cache_of`` is the index of an
    *earlier schedule entry* whose cache this run reads instead of writing one of
    its own (``None``: the entry owns a cache of its own).
    """

    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    """Everything the engine needs to build a model, independent of architecture."""

    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: List[int] = field(default_factory=list)
    #: tensors that may be present in a checkpoint without being read
    optional_tensors: List[str] = field(default_factory=list)


def require(d: Dict[str, Any], key: str, typ, where: str = "config.json"):
    """Fetch a required key with a type check; the error names the key.

    The reference's metadata getters fail the same way: "missing metadata key"
    and "... is not an integer/number/string" (skyla-gguf/src/lib.rs:123-141).
    """
    if key not in d:
        raise ConfigError(f"{where}: missing key '{key}'")
    return _typed(d[key], key, typ, where)


def optional(d: Dict[str, Any], key: str, typ, default, where: str = "config.json"):
    if key not in d or d[key] is None:
        return default
    return _typed(d[key], key, typ, where)


def _typed(v, key, typ, where):
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v.is_integer():
                return int(v)
            raise ConfigError(f"{where}: '{key}' is not an integer (got {v!r})")
        return v
    if typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{where}: '{key}' is not a number (got {v!r})")
        return float(v)
    if typ is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"{where}: '{key}' is not a boolean (got {v!r})")
        return v
    if typ is str:
        if not isinstance(v, str):
            raise ConfigError(f"{where}: '{key}' is not a string (got {v!r})")
        return v
    if typ is dict:
        if not isinstance(v, dict):
            raise ConfigError(f"{where}: '{key}' is not an object (got {v!r})")
        return v
    raise TypeError(typ)
