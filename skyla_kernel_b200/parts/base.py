"""What a part is, and the registries that the configuration's part names point into.

A part is built from a :class:`~skyla_kernel_b200.config.PartSpec` (its sizes,
constants and the checkpoint names of its tensors) and a :class:`Runtime` (device
and precision).  It declares its tensors before any weight is read, takes them in
``load`` and then runs inside a step.  A part never looks at the model it is in:
the reference's ``Mixer`` and ``Ffn`` enums (skyla-ref/src/model.rs:17-20,
skyla-ref/src/ffn.rs:6-19) become entries of these tables, so another kind of
mixer, feed-forward, norm, position encoding or block is one ``register_*`` call.

Interfaces (``ctx`` is the step's :class:`~skyla_kernel_b200.engine.batch.StepContext`;
``x`` the float32 residual stream ``[tokens, hidden]``):

* norm           ``forward(ctx, x, out, rows=None)``: ``out[r] = norm(x[rows[r]])``; a norm of
                 the form "one scalar per row times a fixed vector" may say so with
                 ``rms_scale_form()`` (see ``parts/norm.py``), which lets the product before
                 it prepare its input
* mixer          ``cache_need()``, ``state_need()``, ``forward(ctx, h, x, entry)``:
                 adds its output to ``x``; ``entry`` says which cache it uses
* feed-forward   ``forward(ctx, h, x)``: adds its output to ``x``
* position       whatever the mixers that accept it read (rotary: ``tables()``)
* block          ``forward(ctx, x, entry)`` with the four parts above inside
* embedding      ``forward(ctx, tokens, x)``;  head: ``forward(ctx, h, logits)``
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Callable, Dict, Optional

import torch

from ..config.base import ConfigError, PartSpec
from ..weights.loader import TensorDecl


@dataclass
class Runtime:
    """Where and in which precision a model runs.

    ``float32``: weights, cache and activations in 32-bit, plain kernels only.
    ``bfloat16``: 16-bit weights, cache and matrix-product operands; the residual
    stream, norms, softmax, rotation and accumulation stay 32-bit.
    """

    device: torch.device
    dtype: str = "bfloat16"
    #: streaming multiprocessors of the device; asked from the device when not given (a runtime on
    #: a device without them, as the dispatch tests build, has to say which machine it stands for)
    n_sms: Optional[int] = None
    #: {blocks per cluster: clusters of the weight-streaming kernel that run at a time}; asked from the device
    #: when not given
    cluster_room: Optional[dict] = None

    def __post_init__(self):
        if self.dtype in ("fp32", "float"):
            self.dtype = "float32"
        if self.dtype in ("bf16",):
            self.dtype = "bfloat16"
        if self.dtype not in ("float32", "bfloat16"):
            raise ValueError(f"dtype must be float32 or bfloat16, not {self.dtype!r}")
        self.device = torch.device(self.device)
        self._placed = {}
        self.shared_parts = {}
        self._kernel_state = None

    @property
    def sm_count(self) -> int:
        if self.n_sms is None:
            if self.device.type != "cuda":
                raise ValueError("a runtime that is not on a CUDA device must be given its number of SMs")
            self.n_sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        return self.n_sms

    @property
    def clusters(self) -> dict:
        if self.cluster_room is None:
            if self.device.type != "cuda":
                raise ValueError("a runtime that is not on a CUDA device must be given its room for clusters")
            from ..kernels.ops import rows_cluster_room
            self.cluster_room = rows_cluster_room(self.device)
        return self.cluster_room

    @property
    def kernel_state(self):
        """What this runtime's kernels keep between launches (error word, counters, scratch): one per
        runtime, that is per engine, so that two engines on one device share nothing."""
        if self._kernel_state is None:
            from ..kernels.ops import KernelState
            self._kernel_state = KernelState(self.device)
        return self._kernel_state

    def forget_host_tensors(self) -> None:
        """Drop the host-to-device placement table once a model is loaded."""
        self._placed = {}

    @property
    def full_precision(self) -> bool:
        return self.dtype == "float32"

    @property
    def act_dtype(self) -> torch.dtype:
        return torch.float32 if self.full_precision else torch.bfloat16

    @property
    def cache_dtype(self) -> torch.dtype:
        return self.act_dtype

    def matrix(self, t: torch.Tensor, shared: bool = False) -> torch.Tensor:
        """A weight matrix on the device in the precision of this runtime.

        In 32-bit mode everything is widened (exactly).  In bfloat16 mode a
        matrix stored in 16 bits stays bfloat16 and one stored in 32 bits stays
        32-bit; the matrix products take either.  ``shared``: the same stored
        tensor may be asked for by two parts (a tied head and the embedding) and
        is then placed once; the host tensor is kept alive until the model is
        loaded so that its identity cannot be taken by another tensor.
        """
        if shared and id(t) in self._placed:
            return self._placed[id(t)][1]
        if self.full_precision:
            placed = t.to(device=self.device, dtype=torch.float32).contiguous()
        else:
            placed = t.to(device=self.device).contiguous()
        if shared:
            self._placed[id(t)] = (t, placed)
        return placed

    def vector(self, t: torch.Tensor) -> torch.Tensor:
        """A norm weight or other small table: always 32-bit on the device."""
        return t.to(device=self.device, dtype=torch.float32).contiguous()


class Part:
    """Base of all parts."""

    #: CUDA source modules (csrc/<name>.cu) the part launches, compiled before first use
    kernel_modules = ()
    #: True if forward() only launches kernels on the current stream and never reads
    #: device memory on the host, so that a step may be captured in a CUDA graph
    graph_safe = False
    #: :class:`StepPlan` objects: what the part wants worked out on the host once a step
    step_plans = ()

    def __init__(self, spec: PartSpec, rt: Runtime):
        self.spec = spec
        self.rt = rt

    @classmethod
    def declare(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        """Checkpoint name -> shape and kind of every tensor the part reads."""
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Take the declared tensors (as stored, on the host or already on the device) and keep what
        the kernels need.  A part that copies tensors into a fused matrix of its own may remove them
        from ``tensors`` (``pop``) so that the originals can be freed; a tensor that another part may
        also declare (a tied head) stays."""

    def kernels_needed(self):
        return tuple(self.kernel_modules)

    def weight_bytes(self) -> int:
        return 0


class StepPlan:
    """Integers that a part wants worked out on the host once a step, from the positions of the step's
    sequences, and sent to the device with the step's other arrays (one copy): work lists and the like
    that are the same for every layer with the same need.  A part lists its plans in ``step_plans``;
    plans with equal ``key`` are one plan, which the parts find as ``ctx.plans[key]`` (int32, on the
    device, 16-byte aligned; absent where the step's builder was not given the plan).
    """

    key = None

    def size(self, n_seqs: int, pages_width: int, decode: bool) -> int:
        """Ints the plan takes for a step of ``n_seqs`` sequences whose page lists have ``pages_width``
        columns (0: none for such a step); ``decode``: every sequence brings one token.  The size may
        depend on nothing else, so that a recorded step keeps its layout."""
        return 0

    def fill(self, out, starts, ns, page_size: int) -> None:
        """Write the plan into ``out`` (int32 NumPy, ``size`` ints) for sequences that hold ``starts[b]``
        positions and bring ``ns[b]`` new tokens."""


class NormedInput:
    """The input of a mixer or feed-forward before it is computed: ``norm(x)``.

    A block hands this to parts that set ``takes_normed_input = True``; such a part either
    calls :meth:`tensor` (the norm runs as a kernel of its own) or, where the product that
    wrote ``x`` last prepared the norm's input (:attr:`ahead`), feeds that to its first product.
    Parts without the flag get ``tensor()``.
    """

    def __init__(self, ctx, x: torch.Tensor, norm):
        self.ctx, self.x, self.norm = ctx, x, norm
        self._tensor = None
        #: (x * norm.weight in bfloat16, shares of the rows' sums of squares) where the product that
        #: wrote ``x`` last left them (``Linear.forward(..., ctx=ctx)``); a part may feed them to its
        #: first product (``scale_in=``) instead of calling :meth:`tensor`
        self.ahead = ctx.take_ahead(norm, x) if hasattr(ctx, "take_ahead") else None

    def tensor(self) -> torch.Tensor:
        if self._tensor is None:
            ctx, x = self.ctx, self.x
            h = ctx.buffer("block.normed", (ctx.n_tokens, x.shape[1]), ctx.rt.act_dtype)
            self.norm.forward(ctx, x, h)
            ctx.mark("rmsnorm")
            self._tensor = h
        return self._tensor


_REGISTRIES: Dict[str, Dict[str, type]] = {
    k: {} for k in ("norm", "mixer", "feed_forward", "position", "block", "embedding", "head")}


def _register(category: str, kind: str, cls: type) -> type:
    _REGISTRIES[category][kind] = cls
    return cls


def register_norm(kind: str, cls: type) -> type: return _register("norm", kind, cls)
def register_mixer(kind: str, cls: type) -> type: return _register("mixer", kind, cls)
def register_feed_forward(kind: str, cls: type) -> type: return _register("feed_forward", kind, cls)
def register_position(kind: str, cls: type) -> type: return _register("position", kind, cls)
def register_block(kind: str, cls: type) -> type: return _register("block", kind, cls)
def register_embedding(kind: str, cls: type) -> type: return _register("embedding", kind, cls)
def register_head(kind: str, cls: type) -> type: return _register("head", kind, cls)


def part_class(category: str, kind: str) -> type:
    try:
        return _REGISTRIES[category][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES[category])) or "(none)"
        raise ConfigError(f"no {category.replace('_', '-')} part named {kind!r}; registered: {known}") from None


def build_part(category: str, spec: PartSpec, rt: Runtime):
    """Build a part; a class marked ``shareable`` is built once per runtime and parameter set."""
    cls = part_class(category, spec.kind)
    if getattr(cls, "shareable", False):
        key = (category, spec.kind, json.dumps(spec.params, sort_keys=True, default=str))
        if key not in rt.shared_parts:
            rt.shared_parts[key] = cls(spec, rt)
        return rt.shared_parts[key]
    return cls(spec, rt)


def declare_part(category: str, spec: PartSpec) -> Dict[str, TensorDecl]:
    return part_class(category, spec.kind).declare(spec)
