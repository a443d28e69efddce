"""Greedy, temperature, top-k and top-p sampling."""
from .sampler import CHAT_DEFAULTS, Sampler, SamplingParams

__all__ = ["CHAT_DEFAULTS", "Sampler", "SamplingParams"]
