"""One registry from an architecture's name to its configuration class.

The reference gates on ``general.architecture`` with a string match and fails
with "unsupported architecture" otherwise (skyla-ref/src/lib.rs:79-83).  Here
the name is ``architectures[0]`` of config.json; a configuration class turns the
file's keys into a :class:`~.base.ModelSpec`, which is all the engine sees.
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, Protocol

from .base import ConfigError, ModelSpec


class ArchitectureConfig(Protocol):
    """What a configuration class must offer to be registered."""

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ArchitectureConfig": ...

    def to_dict(self) -> Dict[str, Any]: ...

    def to_spec(self) -> ModelSpec: ...


_ARCHITECTURES: Dict[str, Any] = {}


def register_architecture(name: str, config_cls) -> None:
    """Make ``config_cls`` the reader of config.json files whose architecture is ``name``."""
    for attr in ("from_dict", "to_spec"):
        if not hasattr(config_cls, attr):
            raise TypeError(f"configuration class for {name!r} lacks {attr}()")
    _ARCHITECTURES[name] = config_cls


def registered_architectures():
    return sorted(_ARCHITECTURES)


def architecture_name(d: Dict[str, Any]) -> str:
    archs = d.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: missing key 'architectures' (a list with the model class name)")
    return archs[0]


def config_from_dict(d: Dict[str, Any]):
    name = architecture_name(d)
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unsupported architecture {name!r}; registered: "
                          f"{', '.join(registered_architectures()) or '(none)'}")
    return _ARCHITECTURES[name].from_dict(d)


def config_from_folder(folder: str):
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{folder}: no config.json")
    with open(path) as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level is not an object")
    return config_from_dict(d)
