"""skyla_kernel_b200: a one-GPU generation library for the Qwen3 dense decoder on
NVIDIA B200 (sm_100a), in the shape of maulanasdqn/skyla-kernel.

    import skyla_kernel_b200 as skyla
    model = skyla.load("model_dir", dtype="bfloat16", max_tokens=8192)
    outputs = model.generate([[1, 2, 3], [4, 5]], max_new_tokens=16)
"""
from .api import Model, load
from .config import (ConfigError, Qwen3Config, config_from_dict, config_from_folder,
                     register_architecture)
from .engine import Engine, StepItem
from .sampling import SamplingParams
from .weights import WeightError, write_model_folder

__all__ = ["Model", "load", "ConfigError", "Qwen3Config", "config_from_dict", "config_from_folder",
           "register_architecture", "Engine", "StepItem", "SamplingParams", "WeightError",
           "write_model_folder"]
