"""Weights: safetensors container, name-keyed loader, random-weights mode."""
from .loader import TensorDecl, WeightError, load_weights
from .random_init import random_tensors, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["TensorDecl", "WeightError", "load_weights", "random_tensors", "write_model_folder",
           "SafetensorsError", "SafetensorsFile", "write_safetensors"]
