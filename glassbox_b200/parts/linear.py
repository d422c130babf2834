"""Matrix products: out[M, N] (+)= a[M, K] @ w[N, K]^T, weights row-major [out, in]
(crates/glassbox-core/src/kernels.rs:381, 586).

The kernel is chosen by operand types only: all-float32 operands run the FMA kernel (the true
32-bit path); bfloat16 operands run the tensor-core kernel when the shape allows and the FMA
kernel otherwise. ``accumulate`` adds into a float32 ``out`` (the residual stream).
"""
from __future__ import annotations

import torch

from .. import kernels


def linear(ctx, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and kernels.gemm_tc_supported(a, w, out):
        kernels.gemm_tc(a, w, out, accumulate)
    else:
        kernels.gemm_simt(a, w, out, accumulate)
