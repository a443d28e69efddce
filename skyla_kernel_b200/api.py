"""The Python entry point: ``load`` a model folder (or a configuration with random
weights) and ``generate`` token ids from token ids.

The reference is driven from its ``skyla`` command line and has no tokenizer in
its repository; neither has this library: prompts and results are token ids.
"""
from __future__ import annotations

import os
import tempfile
from typing import Dict, List, Optional, Sequence, Union

import torch

from .config import config_from_dict, config_from_folder
from .engine.batch import StepItem
from .engine.engine import Engine
from .engine.generate import Finished, Request, generate
from .engine.model import declared_tensors
from .sampling import Sampler, SamplingParams
from .weights import random_tensors


class Model:
    """A loaded model with its cache: ``step``, ``generate``, slots."""

    def __init__(self, engine: Engine):
        self.engine = engine
        self.config = engine.config
        self._samplers: Dict[SamplingParams, Sampler] = {}

    # ---- what the generation loop drives
    @property
    def n_pages(self) -> int:
        return self.engine.cache.n_pages

    @property
    def page_size(self) -> int:
        return self.engine.cache.page_size

    @property
    def max_slots(self) -> int:
        return self.engine.cache.max_slots

    def alloc_slot(self) -> int:
        return self.engine.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.engine.free_slot(slot)

    def reset(self, slot: int) -> int:
        """Forget a sequence; returns a fresh, empty slot (the reference's ``reset``,
        skyla-engine/src/engine.rs:82-89)."""
        self.engine.free_slot(slot)
        return self.engine.alloc_slot()

    def step(self, items: Sequence[StepItem]) -> torch.Tensor:
        return self.engine.step(items)

    # ---- generation
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: Union[int, Sequence[int]] = 16,
                 temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0,
                 stop_ids: Optional[Sequence[int]] = None, max_batch: int = 64,
                 emit_stop: bool = False, return_reasons: bool = False, on_step=None):
        """Token ids in, token ids out; one result per prompt, in order.

        ``temperature=0`` is greedy.  ``stop_ids=None`` takes the configuration's
        end-of-sequence ids; pass ``[]`` for none.  ``on_step(step, live)`` is called on
        the host after every step's tokens have arrived (measurement hooks in here).
        """
        params = SamplingParams(temperature, top_k, top_p, seed)
        sampler = self._samplers.get(params)
        if sampler is None:
            sampler = self._samplers[params] = Sampler(params, self.engine.rt.device, self.engine.rt.kernel_state)
        if stop_ids is None:
            stop_ids = self.engine.spec.stop_token_ids
        if isinstance(max_new_tokens, int):
            max_new_tokens = [max_new_tokens] * len(prompts)
        reqs = [Request(list(p), int(n), tuple(stop_ids)) for p, n in zip(prompts, max_new_tokens)]
        backend = _Backend(self, sampler)
        done = generate(backend, reqs, max_batch=max_batch, emit_stop=emit_stop, on_step=on_step)
        if return_reasons:
            return [d.tokens for d in done], [d.reason for d in done]
        return [d.tokens for d in done]


class _Backend:
    def __init__(self, model: Model, sampler: Sampler):
        self.m = model
        self.sampler = sampler
        self.n_pages, self.page_size, self.max_slots = model.n_pages, model.page_size, model.max_slots

    def alloc_slot(self):
        return self.m.alloc_slot()

    def free_slot(self, slot):
        self.m.free_slot(slot)

    def step(self, items):
        return self.m.engine.step(items, borrow=True)  # sampled at once, before the next step

    def sample(self, logits, req_ids, steps) -> List[int]:
        tokens = self.sampler(logits, req_ids, steps).cpu().tolist()
        self.m.engine.check_errors()  # the copy above has waited for the step
        return tokens

    def step_async(self, items, req_ids, steps) -> "_Tokens":
        """Step and sample without waiting: the tokens stay on the device for the next step and
        travel to pinned host memory on the side, the kernels' error word with them."""
        logits = self.m.engine.step(items, borrow=True)
        return _Tokens(self.sampler(logits, req_ids, steps), self.m.engine.rt.kernel_state)


class _Tokens:
    """A step's sampled tokens: on the device for the next step, and on their way to the host."""

    def __init__(self, device_tokens: torch.Tensor, state):
        self.device_tokens = device_tokens
        self._state = state
        n = device_tokens.numel()
        self._host = torch.empty(n + 1, dtype=torch.int32, pin_memory=True)
        self._host[:n].copy_(device_tokens, non_blocking=True)
        self._host[n:].copy_(state.error_flag, non_blocking=True)
        self._ready = torch.cuda.Event()
        self._ready.record()

    def tokens(self) -> List[int]:
        """Waits for this step; raises ``KernelError`` if a kernel reported a fault up to it."""
        self._ready.synchronize()
        host = self._host.tolist()
        self._state.raise_if(host[-1])
        return host[:-1]


def load(model: Union[str, dict, object], dtype: str = "bfloat16", max_tokens: int = 4096,
         max_slots: Optional[int] = None, device="cuda:0", seed: int = 0,
         linear_std: float = 0.02, norm_std: float = 0.02) -> Model:
    """``model``: a folder with config.json and model.safetensors, or a configuration
    (a dict in config.json form or a configuration object) to fill with seeded
    random weights."""
    if isinstance(model, (str, os.PathLike)):
        return Model(Engine.from_folder(os.fspath(model), dtype, max_tokens, max_slots, device))
    config = config_from_dict(model) if isinstance(model, dict) else model
    store = torch.float32 if dtype in ("float32", "fp32") else torch.bfloat16
    tensors = random_tensors(declared_tensors(config.to_spec()), seed, store, linear_std, norm_std)
    return Model(Engine(config, tensors, dtype, max_tokens, max_slots, device))
