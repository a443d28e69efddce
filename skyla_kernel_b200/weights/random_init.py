"""Random-weights mode: a model folder from a configuration and a seed.

The reference has no such mode (it only reads checkpoints); measurements and
tests here need models of every size without a network.  Matrices and embeddings
are drawn from N(0, linear_std), norm weights from 1 + N(0, norm_std); each
tensor has a stream of its own, keyed by the seed and the tensor's name, so the
values of one tensor do not depend on which other tensors the model has.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict

import torch

from .loader import TensorDecl
from .safetensors_io import write_safetensors


def _generator(seed: int, name: str) -> torch.Generator:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF)
    return g


def random_tensors(expected: Dict[str, TensorDecl], seed: int, dtype: torch.dtype = torch.bfloat16,
                   linear_std: float = 0.02, norm_std: float = 0.02) -> Dict[str, torch.Tensor]:
    out = {}
    for name, decl in expected.items():
        g = _generator(seed, name)
        if decl.init == "int":
            out[name] = torch.randint(0, 8, decl.shape, generator=g, dtype=torch.int32)
            continue
        t = torch.randn(decl.shape, generator=g, dtype=torch.float32)
        t = t * linear_std if decl.init == "linear" else 1.0 + t * norm_std
        out[name] = t.to(dtype)
    return out


def write_model_folder(folder: str, config, seed: int, dtype: str = "bfloat16",
                       linear_std: float = 0.02, norm_std: float = 0.02) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` into ``folder``.

    ``config`` is any registered configuration object (``to_dict``, ``to_spec``).
    """
    from ..engine.model import declared_tensors  # late: engine imports weights
    tdt = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[dtype]
    os.makedirs(folder, exist_ok=True)
    d = config.to_dict()
    d["torch_dtype"] = dtype
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(d, f, indent=1)
    tensors = random_tensors(declared_tensors(config.to_spec()), seed, tdt, linear_std, norm_std)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      {"format": "pt", "seed": str(seed)})
    return folder
