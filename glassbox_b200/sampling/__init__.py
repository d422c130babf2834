"""Turning logits into the next token."""
from .sampler import Rng, Sampler, SamplerConfig, argmax_first

__all__ = ["Rng", "Sampler", "SamplerConfig", "argmax_first"]
