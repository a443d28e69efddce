"""Rotary position encoding, rotate-half ("NeoX") pairing, as tables.

``f_i = theta^(-2i/d)`` for ``i < d/2`` with ``d = n_rot``; the angle of position
``p`` is the 32-bit product ``p * f_i``; element pairs ``(u_i, u_{i+d/2})`` turn
by it (skyla-ref/src/rope.rs:37-41,59-68).  Optional YaRN scaling blends the
frequencies and scales cos and sin by ``mscale`` (rope.rs:43-57, BETA_FAST=32,
BETA_SLOW=1 at rope.rs:4-5).  The part owns one ``[positions, d/2]`` table of cos
and one of sin, built once on the host (sine and cosine of the 32-bit angle are
taken in 64-bit and rounded once) and read by the kernels, so rotation angles
are the same numbers in every kernel and every precision.
"""
from __future__ import annotations

import math
from typing import Dict, Tuple

import torch

from .base import Part, register_position

_BETA_FAST, _BETA_SLOW = 32.0, 1.0


def rotary_frequencies(n_rot: int, theta: float, scaling=None) -> Tuple[torch.Tensor, float]:
    """32-bit frequencies ``[n_rot/2]`` and the cos/sin multiplier."""
    d = torch.tensor(float(n_rot), dtype=torch.float32)
    i = torch.arange(n_rot // 2, dtype=torch.float32)
    base = torch.pow(torch.tensor(float(theta), dtype=torch.float32), -2.0 * i / d)
    if not scaling:
        return base, 1.0
    factor = float(scaling["factor"])
    orig = float(scaling["original_max_position_embeddings"])
    attn_factor = float(scaling.get("attn_factor", 1.0))

    def corr(beta: float) -> float:
        return n_rot * math.log(orig / (beta * 2.0 * math.pi)) / (2.0 * math.log(theta))

    fs = 1.0 / factor
    low = max(math.floor(corr(_BETA_FAST)), 0.0)
    high = min(math.ceil(corr(_BETA_SLOW)), n_rot - 1.0)
    y = (i - low) / max(high - low, 0.001)
    mix = 1.0 - y.clamp(0.0, 1.0)
    freqs = base * (fs * (1.0 - mix) + mix)
    mscale = attn_factor * (1.0 + 0.1 * math.log(1.0 / fs))
    return freqs.to(torch.float32), float(mscale)


class RotaryNeox(Part):
    """Parameters: ``n_rot`` (leading elements of a head that rotate), ``theta``,
    ``max_positions`` (first table size; it grows when a step goes further),
    ``scaling`` (``None`` or the YaRN numbers).  Layers with the same parameters
    share one instance (``shareable``)."""

    shareable = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.n_rot = int(spec.params["n_rot"])
        if self.n_rot % 2:
            raise ValueError("rotary width must be even")
        self.theta = float(spec.params["theta"])
        self.scaling = spec.params.get("scaling")
        self.freqs, self.mscale = rotary_frequencies(self.n_rot, self.theta, self.scaling)
        self.cos = self.sin = None
        self.version = 0
        self._retired = []  # earlier, shorter tables stay valid for whoever captured their address
        self._grow(max(1, int(spec.params.get("max_positions", 1))))

    def _grow(self, n: int) -> None:
        if self.cos is not None:
            self._retired.append((self.cos, self.sin))
        pos = torch.arange(n, dtype=torch.float32)
        ang = (pos[:, None] * self.freqs[None, :]).to(torch.float64)  # the product itself is 32-bit
        self.cos = (torch.cos(ang) * self.mscale).to(torch.float32).to(self.rt.device).contiguous()
        self.sin = (torch.sin(ang) * self.mscale).to(torch.float32).to(self.rt.device).contiguous()
        self.version += 1

    def tables(self, n_positions: int):
        """(cos, sin, n_rot) covering positions ``0 .. n_positions-1``."""
        if n_positions > self.cos.shape[0]:
            n = self.cos.shape[0]
            while n < n_positions:
                n *= 2
            self._grow(n)
        return self.cos, self.sin, self.n_rot


class NoPosition(Part):
    """No position encoding inside the mixer."""

    def tables(self, n_positions: int):
        return None, None, 0


register_position("rotary_neox", RotaryNeox)
register_position("none", NoPosition)
