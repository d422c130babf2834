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
from .base import DeferredNorm, PreparedNorm


def weights_ahead(ctx, w: torch.Tensor):
    """The weight matrix that the step will use two products from now (or None while unknown)."""
    order = getattr(ctx, "weight_order", None)
    return order.ahead(w) if order is not None else None


def _resolve(a, w=None):
    """(tensor, norm or None, deferred or None, row scale or None) for an input that may be a ``DeferredNorm``
    in front of a product with ``w``:
    the residual rows with the norm that the stream kernel applies on the way in (few rows); or the rows that the
    product before prepared, with the scale that a tile kernel applies on the way out; or the normalised rows."""
    if isinstance(a, DeferredNorm):
        rms = a.norm.as_rms()
        if rms is not None and a._tensor is None and (
                kernels.stream_folds(a.x.shape[0], w) if w is not None else a.x.shape[0] <= kernels.STREAM_FUSE_MAX_ROWS):
            return a.x, rms, a, None
        ready = a.prepared()
        if ready is not None:
            return ready[0], None, a, ready[1]
        return a.tensor(), None, None, None
    return a, None, None, None


def _prepare_next_norm(ctx, out: torch.Tensor, k: int):
    """(gain, pre, ss) for a tile-kernel product that adds into ``out``, if the wiring has said which norm reads
    ``out`` next and that norm is a plain RMSNorm over these columns; else None."""
    norm = getattr(ctx, "next_norm", None)
    rms = norm.as_rms() if norm is not None else None
    rows, n = out.shape
    if rms is None or rms[0].numel() != n or rms[0].dtype != torch.float32 or n % 8:
        return None
    pre = ctx.scratch("h_pre", (rows, n), torch.bfloat16)
    widest = -(-n // 64)     # the narrowest tile gives the most partial sums; the buffer never has to grow
    parts = kernels.gemm_tc_column_tiles(rows, n, k)
    ss = ctx.scratch("h_ss", (rows, widest), torch.float32).view(-1)[:rows * parts].view(rows, parts)
    return norm, rms, pre, ss


def _tile_kernel_wins(rows: int, w: torch.Tensor) -> bool:
    """With few rows the weight-streaming kernel is the fast one, except where one strip of 16 outputs
    per block makes thousands of blocks that each stage all rows again: a very wide matrix (the head)
    with more than 16 rows, or a large one with more than 32. Measured at 64 rows: 49152 x 576, 28 us
    against 93 us; 6144 x 2048, 16 us against 33 us; but 2048 x 8192, 43 us against 33 us (few tiles,
    long k) and everything smaller stays with the streaming kernel."""
    n, k = w.shape
    return (rows > 16 and n >= 16384) or (rows > 32 and n >= 4096 and k >= 1024)


def linear(ctx, a, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """``a`` is a tensor or a ``DeferredNorm``; the latter is folded into the weight-streaming kernel
    when that kernel runs, and computed first otherwise."""
    x, norm, deferred, scale = _resolve(a, w)
    if accumulate:
        ctx.prepared_norm = None      # ``out`` changes: what was prepared from its old values is void
    if scale is not None:
        if kernels.gemm_tc_supported(x, w, out):
            kernels.gemm_tc(x, w, out, accumulate, ctx.status, row_scale=scale)
            return
        x, scale = deferred.tensor(), None
    wide = norm is None and _tile_kernel_wins(x.shape[0], w) and kernels.gemm_tc_supported(x, w, out)
    if not wide and kernels.gemm_stream_supported(x, w) and (norm is not None or x.dtype == torch.bfloat16):
        kernels.gemm_stream(x, w, out, accumulate, norm=norm, prefetch=weights_ahead(ctx, w))
        return
    if deferred is not None:
        x = deferred.tensor()
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and kernels.gemm_tc_supported(x, w, out):
        nxt = _prepare_next_norm(ctx, out, x.shape[1]) if accumulate else None
        if nxt is not None:
            next_norm, (gain, eps), pre, ss = nxt
            kernels.gemm_tc(x, w, out, True, ctx.status, prepare=(gain, pre, ss))
            ctx.prepared_norm = PreparedNorm(next_norm, out, pre, kernels.RowScale(ss, eps))
        else:
            kernels.gemm_tc(x, w, out, accumulate, ctx.status)
    else:
        kernels.gemm_simt(x, w, out, accumulate)


def gated_linear(ctx, a, w_gate_up: torch.Tensor, act: torch.Tensor) -> bool:
    """act = silu(a Wgate^T) * (a Wup^T) in one kernel when the shape allows; returns False (and
    does nothing) otherwise, and the caller runs the product and the activation separately."""
    inter = w_gate_up.shape[0] // 2
    x, norm, _, scale = _resolve(a, w_gate_up)
    if scale is not None:
        if (w_gate_up.dtype == torch.bfloat16 and act.dtype == torch.bfloat16
                and kernels.gemm_tc_supported(x, w_gate_up, act)):
            kernels.gemm_tc_gated(x, w_gate_up, act, ctx.status, row_scale=scale)
            return True
        x = a.tensor()
    tiles = (x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and act.dtype == torch.bfloat16
             and kernels.gemm_tc_supported(x, w_gate_up, act))
    wide = norm is None and tiles and _tile_kernel_wins(x.shape[0], w_gate_up)
    if (not wide and kernels.gemm_stream_supported(x, w_gate_up) and (norm is not None or x.dtype == torch.bfloat16)
            and inter % 16 == 0 and act.dtype == torch.bfloat16):
        kernels.gemm_stream(x, w_gate_up, act, gated=True, norm=norm, prefetch=weights_ahead(ctx, w_gate_up))
        return True
    if isinstance(a, DeferredNorm):
        x = a.tensor()
    if wide or (tiles and x.shape[0] > kernels.STREAM_MAX_ROWS):
        kernels.gemm_tc_gated(x, w_gate_up, act, ctx.status)
        return True
    return False
