"""What the measurements share: the layer sizes they are quoted on and a model of such sizes with
seeded random weights drawn on the device (no checkpoint of that size has to exist anywhere).

The reference quotes its numbers on Qwen3 0.6B, 4B and 8B checkpoints (README.md:25-54); here the
sizes are data of the measurement, not of the library: no part and no kernel knows them.
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

# layer sizes of the Qwen3 dense models that the measurements name
QWEN3_8B = dict(hidden_size=4096, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
                head_dim=128, intermediate_size=12288, vocab_size=151936, rope_theta=1000000.0,
                rms_norm_eps=1e-6, max_position_embeddings=40960, tie_word_embeddings=False)
QWEN3_4B = dict(QWEN3_8B, hidden_size=2560, intermediate_size=9728, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600)
SHAPES = {"8b": QWEN3_8B, "4b": QWEN3_4B, "32b": QWEN3_32B}


def random_config(shape: Union[str, dict], layers: Optional[int] = None):
    from .config import Qwen3Config
    base = dict(SHAPES[shape] if isinstance(shape, str) else shape)
    if layers:
        base["num_hidden_layers"] = layers
    return Qwen3Config(**base)


def random_tensors_on_device(cfg, seed: int = 0, store: torch.dtype = torch.bfloat16, device="cuda:0",
                             linear_std: float = 0.02, norm_std: float = 0.02):
    """The model's tensors by checkpoint name, drawn on the device: N(0, linear_std), norm weights
    1 + N(0, norm_std), each tensor from a stream of its own."""
    from .engine import declared_tensors
    from .kernels import ops
    tensors = {}
    for i, (name, d) in enumerate(declared_tensors(cfg.to_spec()).items()):
        t = torch.empty(d.shape, dtype=store, device=device)
        if d.init == "norm":
            ops.fill_normal(t, 1.0, norm_std, seed * 100003 + i)
        else:
            ops.fill_normal(t, 0.0, linear_std, seed * 100003 + i)
        tensors[name] = t
    return tensors


def random_engine(shape: Union[str, dict], layers: Optional[int] = None, max_tokens: int = 4096,
                  max_slots: Optional[int] = None, seed: int = 0, dtype: str = "bfloat16", device="cuda:0",
                  linear_std: float = 0.02, norm_std: float = 0.02):
    """(engine, configuration) of a model with the layer sizes of ``shape`` (a key of ``SHAPES`` or a
    config.json-style dict) and ``layers`` layers (default: the shape's own), with random weights."""
    from .engine import Engine
    cfg = random_config(shape, layers)
    store = torch.float32 if dtype in ("float32", "fp32") else torch.bfloat16
    tensors = random_tensors_on_device(cfg, seed, store, device, linear_std, norm_std)
    engine = Engine(cfg, tensors, dtype, max_tokens=max_tokens, max_slots=max_slots, device=device)
    del tensors
    torch.cuda.empty_cache()
    return engine, cfg
