"""Interfaces of the parts a layer is put together from, and the registry that builds them.

A part is built from its spec alone (sizes and constants are the spec's fields), declares the
parameters it needs, receives them once, and is then called with a ``StepContext`` that carries
the batch. No part knows which model it sits in, which layer it is, or what its neighbours are.

Interfaces (``ctx`` is ``glassbox_b200.engine.context.StepContext``):

* Embedding: ``forward(ctx, tokens, x)``: ``tokens`` int32 [n] on the device; writes the float32 residual rows
             ``x`` [n, d] (padding rows carry token 0 and are ignored downstream).
* Head:      ``forward(ctx, hs, logits)``: ``hs`` [w, d] (activation dtype, already normed), writes float32
             ``logits`` [w, vocab].
* Norm:      ``forward(ctx, x, out, rows=None)``: ``x`` float32 [n, d] residual stream, ``out``
             [m, d] in the activation dtype; ``rows`` (int32 [m]) picks input rows.
* Position:  ``fused_table(device)`` -> float32 [max_position, rotary_dim/2, 2] of (cos, sin) that
             the attention mixer's fused kernel applies, or None; ``rotary_dim``;
             ``apply_qk(ctx, qkv, num_heads, num_kv_heads, head_dim)`` for encodings that are
             not a rotation table (runs before keys are stored).
* Mixer:     ``cache_spec()`` -> ``PagedKvSpec`` | ``StateSpec`` | None;
             ``forward(ctx, h, residual, cache, writes_cache)``: reads ``h`` [n, d] (activation
             dtype), ADDS its output into ``residual`` (float32 [n, d]). ``cache`` is the view of
             the cache layer the schedule assigned to this run.
* FeedForward: ``forward(ctx, h, residual)``: same contract, no cache.

Registering a new part: subclass the interface, give the spec dataclass a fresh ``kind`` string,
and call ``register_part(role, kind, cls)``. Nothing else in the framework changes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Tuple

import torch

from ..weights.binding import ParamSpec


@dataclass(frozen=True)
class PagedKvSpec:
    """A mixer that keeps keys and values per token, in pages. Layers with equal specs share a
    cache group (one block table, one page pool). ``window`` None keeps every token; an integer
    keeps only the last ``window`` tokens, and pages behind the window are given back."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """A mixer that keeps a fixed-size state per request, in a slot: ``shape`` per request,
    zeroed when the request is admitted, overwritten in place each step."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    #: True when every piece of device work this part does is a call into ``glassbox_b200.kernels``. Only then may
    #: its calls be recorded into a decode program and run later, in order, by one persistent kernel; a part that
    #: also enqueues work of its own (torch operations, other libraries) keeps the default and always runs
    #: kernel by kernel.
    launches_through_kernels_only = False

    def recordable(self, decode_only: bool) -> bool:
        """Whether a step through this part can be recorded once and replayed as a CUDA graph (``decode_only``: a step
        in which every request brings exactly one row). It can when the part reads everything that changes from step
        to step (tokens, positions, slots, block tables, state slots: the tensors of ``ctx``) on the device, and
        nothing of it on the host (``ctx.seqs``, Python numbers taken from tensors). Parts that cannot say False
        and their model's steps of that kind are launched kernel by kernel."""
        return True

    def __init__(self, spec: Any):
        self.spec = spec
        self.params: Dict[str, torch.Tensor] = {}

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        """Receive the loaded parameters (keys are the local names of ``param_specs``)."""
        self.params = dict(params)

    def sub_parts(self) -> Dict[str, "Part"]:
        """Parts this part owns (their parameters are loaded under ``<name>.``)."""
        return {}


class Norm(Part):
    def forward(self, ctx, x, out, rows=None) -> None:
        raise NotImplementedError

    def as_rms(self):
        """(gain, eps) if this norm is a plain RMSNorm that a GEMM kernel may apply on the way in, else
        None (the norm then always runs as its own kernel)."""
        return None


class PreparedNorm:
    """What the product that last added into the residual ``x`` left behind for the norm that reads ``x`` next
    (``ctx.next_norm``, a hint from whoever wires the parts): ``pre`` = bfloat16(x * gain) and the scale that
    completes the norm in the epilogue of the product that consumes it. Valid only while ``x`` is what that
    product wrote: same storage, same version counter (every torch operation in place raises it), and no
    ``linear(..., accumulate=True)`` into it since (which replaces or clears this record)."""
    __slots__ = ("norm", "x_ptr", "version", "rows", "pre", "scale")

    def __init__(self, norm, x: torch.Tensor, pre: torch.Tensor, scale):
        self.norm, self.x_ptr, self.version, self.rows = norm, x.data_ptr(), x._version, x.shape[0]
        self.pre, self.scale = pre, scale

    def matches(self, norm, x: torch.Tensor) -> bool:
        return (self.norm is norm and self.x_ptr == x.data_ptr() and self.version == x._version
                and self.rows == x.shape[0])


class DeferredNorm:
    """The normalised input of a mixer or feed-forward, not yet computed. A part that sets
    ``accepts_deferred_input`` receives this instead of a tensor and hands it to ``linear``, which
    folds the norm into the product (few rows, RMSNorm), or takes what the product before prepared
    (``prepared()``), or calls ``tensor()``; a part that needs the activations themselves calls
    ``tensor()`` and gets them (computed once)."""

    def __init__(self, ctx, norm: "Norm", x: torch.Tensor, name: str = "h"):
        self.ctx, self.norm, self.x, self.name = ctx, norm, x, name
        self._tensor = None
        self.shape = x.shape

    def prepared(self):
        """(bfloat16(x * gain), row scale) if the product that wrote ``x`` prepared this norm, else None."""
        p = getattr(self.ctx, "prepared_norm", None)
        if p is not None and self._tensor is None and p.matches(self.norm, self.x):
            return p.pre, p.scale
        return None

    def tensor(self) -> torch.Tensor:
        if self._tensor is None:
            self._tensor = self.ctx.scratch(self.name, tuple(self.x.shape))
            self.norm.forward(self.ctx, self.x, self._tensor)
        return self._tensor


class Position(Part):
    rotary_dim: int = 0

    def fused_table(self, device) -> Optional[torch.Tensor]:
        return None

    def apply_qk(self, ctx, qkv, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        return None


class Mixer(Part):
    #: set by parts whose ``forward`` can take a ``DeferredNorm`` as ``h``
    accepts_deferred_input = False

    def cache_spec(self):
        return None

    def forward(self, ctx, h, residual, cache, writes_cache: bool) -> None:
        raise NotImplementedError

    def prefetch(self, ctx, cache) -> None:
        """A hint, given while an earlier layer still runs (on another stream): this mixer will soon
        read ``cache``. It may start moving data towards the chip; it must not write anything."""
        return None


class FeedForward(Part):
    accepts_deferred_input = False

    def forward(self, ctx, h, residual) -> None:
        raise NotImplementedError


class TokenEmbedding(Part):
    def forward(self, ctx, tokens, x) -> None:
        raise NotImplementedError


class OutputHead(Part):
    def forward(self, ctx, hs, logits) -> None:
        raise NotImplementedError


ROLES = ("norm", "position", "mixer", "ffn", "arrangement", "embedding", "head")
_REGISTRY: Dict[str, Dict[str, Callable[..., Any]]] = {r: {} for r in ROLES}


def register_part(role: str, kind: str, factory: Callable[..., Any], *, replace: bool = False) -> None:
    """``factory(spec, hidden_size=...)`` builds the part for a spec whose ``kind`` is ``kind``."""
    if role not in _REGISTRY:
        raise ValueError(f"unknown part role {role!r}; roles: {', '.join(ROLES)}")
    if kind in _REGISTRY[role] and not replace:
        raise ValueError(f"{role} {kind!r} is already registered")
    _REGISTRY[role][kind] = factory


def build_part(role: str, spec: Any, **kwargs):
    kind = getattr(spec, "kind", None) if not isinstance(spec, str) else spec
    try:
        factory = _REGISTRY[role][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY[role])) or "(none)"
        raise ValueError(f"no {role} part registered for kind {kind!r}; registered: {known}") from None
    return factory(spec, **kwargs)


def registered(role: str):
    return sorted(_REGISTRY[role])
