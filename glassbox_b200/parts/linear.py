"""Matrix products: out[M, N] (+)= a[M, K] @ w[N, K]^T, weights row-major [out, in]
(crates/glassbox-core/src/kernels.rs:381, 586).

The kernel is chosen by operand types only: all-float32 operands run the FMA kernel (the true
32-bit path); bfloat16 operands run the tensor-core kernel when the shape allows and the FMA
kernel otherwise; with at most 64 rows (decoding) they run the weight-streaming kernel.
``accumulate`` adds into a float32 ``out`` (the residual stream).
"""
from __future__ import annotations

import torch

from .. import kernels


def linear(ctx, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    if kernels.gemm_stream_supported(a, w):
        kernels.gemm_stream(a, w, out, accumulate)
    elif a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and kernels.gemm_tc_supported(a, w, out):
        kernels.gemm_tc(a, w, out, accumulate, ctx.status)
    else:
        kernels.gemm_simt(a, w, out, accumulate)


def gated_linear(ctx, a: torch.Tensor, w_gate_up: torch.Tensor, act: torch.Tensor) -> bool:
    """act = silu(a Wgate^T) * (a Wup^T) in one kernel when the shape allows; returns False (and
    does nothing) otherwise, and the caller runs the product and the activation separately."""
    inter = w_gate_up.shape[0] // 2
    if kernels.gemm_stream_supported(a, w_gate_up) and inter % 16 == 0 and act.dtype == torch.bfloat16:
        kernels.gemm_stream(a, w_gate_up, act, gated=True)
        return True
    return False
