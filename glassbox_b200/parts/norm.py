"""RMSNorm: out_j = w_j * (x_j / sqrt(mean(x^2) + eps)), statistics in float32, no mean
subtraction, no bias, the gain used as stored (crates/glassbox-core/src/model.rs:94-100)."""
from __future__ import annotations

from .. import kernels
from ..weights.binding import ParamSpec
from .base import Norm, register_part


class RmsNorm(Norm):
    launches_through_kernels_only = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        self.eps = float(spec.eps)
        self.hidden_size = hidden_size

    def param_specs(self):
        return {"weight": ParamSpec((self.hidden_size,), role="gain")}

    def forward(self, ctx, x, out, rows=None) -> None:
        kernels.rmsnorm(x, self.params["weight"], out, self.eps, rows)

    def as_rms(self):
        return self.params["weight"], self.eps


register_part("norm", "rmsnorm", RmsNorm, replace=True)
