"""Typed configurations and the architecture registry."""
from .base import (ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry)
from .qwen3 import ARCHITECTURE as QWEN3_ARCHITECTURE
from .qwen3 import Qwen3Config, RopeScaling
from .registry import (architecture_name, config_from_dict, config_from_folder,
                       register_architecture, registered_architectures)

register_architecture(QWEN3_ARCHITECTURE, Qwen3Config)

__all__ = [
    "ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "Qwen3Config",
    "RopeScaling", "architecture_name", "config_from_dict", "config_from_folder",
    "register_architecture", "registered_architectures", "QWEN3_ARCHITECTURE",
]
