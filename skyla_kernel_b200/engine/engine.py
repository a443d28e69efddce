"""The engine: a loaded model, its cache and the step function.

``Engine.step`` is the one function between a batch of sequences' next tokens
and their logits.  It is what the reference's ``Engine::prefill`` and
``Engine::step`` are for one sequence (skyla-engine/src/engine.rs:137-152): it
runs only the tokens it is given, from the cache that earlier steps left, and
appends to it.  Prompts go in one step, then one token per sequence; any other
cut of the tokens gives the same logits up to rounding.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheError, CacheFull, SequenceCache
from ..config import config_from_folder
from ..kernels import build as kernel_build
from ..parts.base import Runtime
from ..weights import load_weights
from .batch import BatchBuilder, StepItem
from .graphs import DecodeGraphs
from .model import DecoderModel, declared_tensors


class EngineError(RuntimeError):
    pass


def _device(device) -> torch.device:
    dev = torch.device(device)
    if dev.type != "cuda":
        raise EngineError("the engine runs on a CUDA device only; there is no host path")
    if not torch.cuda.is_available():
        raise EngineError("no CUDA device is available; the engine cannot run")
    return dev


class Engine:
    """A model on one GPU with a cache of ``max_tokens`` positions.

    ``max_tokens`` counts the positions held by live sequences, each sequence
    rounded up to a whole page of 64.  ``max_slots`` bounds the live sequences
    (default: one per page).  ``tensors`` (checkpoint name -> tensor) is consumed:
    parts take out of it what they copy into matrices of their own, so that a
    caller who keeps no other reference keeps no second copy of the weights.
    """

    def __init__(self, config, tensors: Dict[str, torch.Tensor], dtype: str = "bfloat16",
                 max_tokens: int = 4096, max_slots: Optional[int] = None, device="cuda:0",
                 cuda_graphs: Optional[bool] = None):
        self.config = config
        self.spec = config.to_spec()
        self.rt = Runtime(_device(device), dtype)
        torch.cuda.set_device(self.rt.device)
        self.model = DecoderModel(self.spec, self.rt)
        kernel_build.build_all(self.model.kernels_needed())
        self.model.load(tensors)
        self.cache = SequenceCache(self.model.kv_needs, self.model.state_needs, max_tokens, max_slots,
                                   self.rt.cache_dtype, self.rt.device)
        self.batcher = BatchBuilder(self.rt, self.cache, self.model.tile_heights(), self.model.step_plans())
        self.vocab_size = self.spec.vocab_size
        if cuda_graphs is None:
            cuda_graphs = os.environ.get("SKYLA_CUDA_GRAPHS", "1") != "0"
        # decode steps of the 16-bit path replay captured graphs; the 32-bit path stays eager
        self.graphs = (DecodeGraphs(self.model, self.rt, self.cache)
                       if cuda_graphs and not self.rt.full_precision and self.model.graph_safe() else None)

    # ---------------------------------------------------------------- loading
    @classmethod
    def from_folder(cls, folder: str, dtype: str = "bfloat16", max_tokens: int = 4096,
                    max_slots: Optional[int] = None, device="cuda:0", cuda_graphs: Optional[bool] = None) -> "Engine":
        config = config_from_folder(folder)
        spec = config.to_spec()
        tensors = load_weights(folder, declared_tensors(spec), spec.optional_tensors)
        return cls(config, tensors, dtype, max_tokens, max_slots, device, cuda_graphs)

    # ------------------------------------------------------------------ slots
    def alloc_slot(self) -> int:
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)

    # ------------------------------------------------------------------- step
    def step(self, items: Sequence[StepItem], taps=None, profile: bool = False,
             borrow: bool = False) -> torch.Tensor:
        """Run the items' tokens as one batch; float32 logits at the wanted places.

        ``borrow=True`` returns the engine's own logits buffer, which the next step
        overwrites (the generation loop and the replay program read it at once);
        otherwise the caller gets a copy.

        Rows are ordered by item, then by the item's ``want`` list.  Raises
        :class:`CacheFull` before anything is launched if the tokens do not fit,
        and ``ValueError`` for a token outside the vocabulary (the reference:
        "token {t} is outside the vocabulary", skyla-engine/src/engine.rs:110-112).
        """
        items = list(items)
        if not items:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.rt.device)
        for it in items:
            if len(it.tokens) == 0:
                raise ValueError(f"slot {it.slot}: a step must bring at least one token")
            if it.device_token is not None:
                continue  # a sampler's output on the device: inside the vocabulary by construction
            arr = np.asarray(it.tokens)
            if arr.dtype.kind not in "iu":
                raise ValueError(f"slot {it.slot}: tokens must be integers")
            if arr.min() < 0 or arr.max() >= self.vocab_size:
                bad = int(arr[(arr < 0) | (arr >= self.vocab_size)][0])
                raise ValueError(f"token {bad} is outside the vocabulary (0..{self.vocab_size - 1})")
        growth = [(it.slot, len(it.tokens)) for it in items]
        self.cache.reserve(growth)
        with torch.cuda.device(self.rt.device):
            if (self.graphs is not None and taps is None and not profile
                    and all(len(it.tokens) == 1 and list(it.want) == [0] for it in items)):
                logits = self.graphs.run(items)
                self.cache.advance(growth)
                return logits if borrow else logits.clone()
            ctx = self.batcher.build(items)
            if profile:
                ctx.marks = []
                ctx.mark("start")
            logits = self.model.forward(ctx, taps)
            if profile:
                self._profile = self._read_marks(ctx.marks)
        self.cache.advance(growth)
        return logits if borrow else logits.clone()

    @staticmethod
    def _read_marks(marks):
        torch.cuda.synchronize()
        total = {}
        for (_, a), (label, b) in zip(marks, marks[1:]):
            total[label] = total.get(label, 0.0) + a.elapsed_time(b) * 1e6
        return sorted(total.items(), key=lambda kv: -kv[1])

    def last_step_profile(self):
        """``[(label, nanoseconds)]`` of the last step run with ``profile=True``, largest first
        (the reference's ``Engine::last_step_profile``, skyla-engine/src/engine.rs:91-96)."""
        return list(getattr(self, "_profile", []))

    def check_errors(self) -> None:
        """Raise ``KernelError`` if one of this engine's kernels reported a fault since the last check:
        a bounded wait that ran out, a row of logits without a token, a token outside the embedding
        table.  It waits for the device.  The generation loop reads the same word with every step's
        tokens; callers of :meth:`step` who never synchronize otherwise call this when they read results."""
        self.rt.kernel_state.check()

    # ------------------------------------------------------------------ facts
    def weight_bytes(self) -> int:
        return self.model.weight_bytes_per_step()

    def device_name(self) -> str:
        return torch.cuda.get_device_name(self.rt.device)
