"""Rotary position encoding.

The table is built on the host exactly as Glassbox computes its angles
(crates/glassbox-core/src/model.rs:102-115): the inverse frequency 1 / theta^(2i/dim) is formed
in float64 and rounded to float32; the angle is the float32 product position * inv_freq; sine
and cosine are evaluated in float64 and rounded to float32. Doing the angle in float32 makes
long positions round "like transformers" (model.rs:106), so it is kept.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import Position, register_part


def rotary_table(theta: float, rotary_dim: int, max_position: int) -> torch.Tensor:
    """float32 [max_position, rotary_dim/2, 2] holding (cos, sin)."""
    half = rotary_dim // 2
    i = np.arange(half, dtype=np.float64)
    inv = (1.0 / np.power(np.float64(theta), 2.0 * i / np.float64(rotary_dim))).astype(np.float32)
    pos = np.arange(max_position, dtype=np.float32)
    angle = (pos[:, None] * inv[None, :]).astype(np.float32)  # float32 multiply
    a64 = angle.astype(np.float64)
    table = np.stack([np.cos(a64).astype(np.float32), np.sin(a64).astype(np.float32)], axis=-1)
    return torch.from_numpy(np.ascontiguousarray(table))


class Rope(Position):
    launches_through_kernels_only = True

    def __init__(self, spec, **_):
        super().__init__(spec)
        if spec.pairing != "half":
            raise ValueError(f"rope pairing {spec.pairing!r} is not supported (only 'half')")
        if spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even")
        self.rotary_dim = spec.rotary_dim
        self._tables = {}

    def fused_table(self, device):
        key = str(device)
        if key not in self._tables:
            self._tables[key] = rotary_table(self.spec.theta, self.spec.rotary_dim, self.spec.max_position).to(device)
        return self._tables[key]


class NoPosition(Position):
    launches_through_kernels_only = True

    def __init__(self, spec=None, **_):
        super().__init__(spec)


register_part("position", "rope", Rope, replace=True)
register_part("position", "none", NoPosition, replace=True)
