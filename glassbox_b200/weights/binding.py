"""How a part parameter is fed from a weights file.

An architecture's ``bind`` function returns ``{parameter path: source}``. A parameter path is
the part's place in the model plus the parameter's local name, e.g. ``layers.3.mixer.wqkv``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class ParamSpec:
    """What a part needs: a shape, a role, and (for stacked matrices) the rows of each piece.

    role "matrix": a GEMM operand, [out, in]; kept in the compute dtype (bfloat16 or float32)
                   unless the file stores it in 32-bit, which is then kept.
    role "gain":   a per-channel vector used in 32-bit arithmetic; always held as float32
                   (widening bfloat16 to float32 is exact, so nothing is lost).
    role "table":  integers; held as int32.
    """
    shape: Tuple[int, ...]
    role: str = "matrix"
    pieces: Optional[Tuple[int, ...]] = None


@dataclass(frozen=True)
class Stacked:
    """The parameter is these file tensors concatenated along dim 0, in this order."""
    names: Tuple[str, ...]


@dataclass(frozen=True)
class Tied:
    """The parameter is the same storage as another parameter (e.g. head = embedding).
    ``ignorable`` names file tensors that may be present and are then not read."""
    path: str
    ignorable: Tuple[str, ...] = ()
