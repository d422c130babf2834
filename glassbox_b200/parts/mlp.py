"""Dense gated feed-forward (SwiGLU): residual += (silu(h Wgate^T) * (h Wup^T)) Wdown^T, gate rows
then up rows stacked in one matrix, SiLU as g / (1 + exp(-g)), no bias
(crates/glassbox-core/src/model.rs:327-344; stacking crates/glassbox-core/src/load.rs:62-65)."""
from __future__ import annotations

from .. import kernels
from ..weights.binding import ParamSpec
from .base import FeedForward, register_part
from .linear import gated_linear, linear


class SwiGlu(FeedForward):
    accepts_deferred_input = True
    launches_through_kernels_only = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        self.hidden_size = hidden_size
        self.inter = spec.intermediate_size

    def param_specs(self):
        d, i = self.hidden_size, self.inter
        return {"w_gate_up": ParamSpec((2 * i, d), pieces=(i, i)), "w_down": ParamSpec((d, i))}

    def forward(self, ctx, h, residual) -> None:
        n = h.shape[0]
        act = ctx.scratch("act", (n, self.inter))
        if not gated_linear(ctx, h, self.params["w_gate_up"], act):
            gate_up = ctx.scratch("gate_up", (n, 2 * self.inter))
            linear(ctx, h, self.params["w_gate_up"], gate_up)
            kernels.swiglu(gate_up, act)
        linear(ctx, act, self.params["w_down"], residual, accumulate=True)


register_part("ffn", "swiglu", SwiGlu, replace=True)
