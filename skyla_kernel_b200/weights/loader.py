"""Weights by tensor name, checked against what the model's parts declare.

The reference asks its container for each tensor by name and fails on the first
one that is missing or not a matrix (skyla-gguf/src/lib.rs:143-145,
skyla-ref/src/matrix.rs:14-28).  Here every part declares the tensors it needs
and their shapes; the loader compares that table with the files once and raises
one error that lists every missing tensor, every unexpected tensor and every
wrong shape.

Storage rule: floating tensors stored in 16 bits are kept in bfloat16, tensors
stored in 32-bit floating point stay 32-bit, integer tables become int32.
"""
from __future__ import annotations

import glob
import json
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightError(ValueError):
    """The files do not hold the tensors the model needs."""


@dataclass(frozen=True)
class TensorDecl:
    """What a part declares about one of its tensors.

    ``init`` tells the random-weights mode how to fill it: ``"linear"`` (normal,
    std ``linear_std``), ``"norm"`` (one plus normal, std ``norm_std``) or
    ``"int"`` (small non-negative integers).
    """

    shape: Tuple[int, ...]
    init: str = "linear"


def _files(folder: str) -> List[str]:
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index) as f:
            names = sorted(set(json.load(f).get("weight_map", {}).values()))
        return [os.path.join(folder, n) for n in names]
    single = os.path.join(folder, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    found = sorted(glob.glob(os.path.join(folder, "*.safetensors")))
    if not found:
        raise WeightError(f"{folder}: no model.safetensors")
    return found


def _keep(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.to(torch.bfloat16)
    if t.dtype in (torch.float32, torch.float64):
        return t.to(torch.float32)
    if t.dtype in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8, torch.bool):
        return t.to(torch.int32)
    raise WeightError(f"unsupported dtype {t.dtype}")


def load_weights(folder: str, expected: Dict[str, TensorDecl],
                 optional_names: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """Read the tensors named in ``expected`` from the safetensors files of ``folder``.

    Returns CPU tensors that own their memory.  ``optional_names`` may be present
    in the files without being used (a stored copy of a tied output matrix).
    """
    try:
        files = [SafetensorsFile(p) for p in _files(folder)]
    except (SafetensorsError, OSError) as e:
        raise WeightError(str(e)) from None
    where: Dict[str, SafetensorsFile] = {}
    for f in files:
        for n in f.names():
            where[n] = f
    optional_names = set(optional_names)
    missing = [n for n in expected if n not in where]
    unexpected = sorted(n for n in where if n not in expected and n not in optional_names)
    wrong = []
    for n, decl in expected.items():
        if n in where:
            dt, shape = where[n].info(n)
            if tuple(shape) != tuple(decl.shape):
                wrong.append(f"{n}: file has {list(shape)}, model needs {list(decl.shape)}")
            elif decl.init == "int" and dt.is_floating_point:
                wrong.append(f"{n}: file has {dt}, model needs an integer table")
            elif decl.init != "int" and not dt.is_floating_point:
                wrong.append(f"{n}: file has {dt}, model needs floating point")
    if missing or unexpected or wrong:
        parts = [f"{folder}: the weight files do not match the model"]
        if missing:
            parts.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            parts.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            parts.append(f"  wrong shape or type ({len(wrong)}): " + "; ".join(wrong))
        raise WeightError("\n".join(parts))
    out = {n: _keep(where[n].tensor(n)).clone() for n in expected}
    for f in files:
        f.close()
    return out
