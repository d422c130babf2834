"""Bind file tensors to part parameters by name, check everything, report everything at once.

Glassbox stops at the first missing tensor and never checks a shape against the config
(crates/glassbox-core/src/load.rs:37-49); this loader collects every missing name, every
unexpected name and every wrong shape and raises one ``WeightsError`` that lists them all.

Precision rule: in bfloat16 mode a matrix is kept in bfloat16 (float16 files are converted),
except that a matrix the file stores in 32-bit stays float32; in float32 mode everything is
widened to float32. Gains are always float32, integer tables int32.
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from .binding import ParamSpec, Tied
from .safetensors_io import SafetensorsFile, WeightsError


def _piece_shapes(spec: ParamSpec, n_pieces: int):
    if n_pieces == 1:
        return [tuple(spec.shape)]
    if spec.pieces is None or len(spec.pieces) != n_pieces or sum(spec.pieces) != spec.shape[0]:
        raise WeightsError(f"binding stacks {n_pieces} tensors but the parameter declares pieces {spec.pieces}")
    return [(rows,) + tuple(spec.shape[1:]) for rows in spec.pieces]


def _target_dtype(spec: ParamSpec, stored, compute_dtype: torch.dtype) -> torch.dtype:
    if spec.role == "table":
        return torch.int32
    if spec.role == "gain":
        return torch.float32
    if compute_dtype == torch.float32:
        return torch.float32
    if any(d in (torch.float32, torch.float64) for d in stored):
        return torch.float32
    return torch.bfloat16


def load_parameters(specs: Dict[str, ParamSpec], binding: dict, st: SafetensorsFile,
                    compute_dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    """Return ``{parameter path: tensor on device}`` or raise one error naming every fault."""
    missing, wrong, unbound = [], [], []
    used, ignorable = set(), set()
    plan = {}
    for path, spec in specs.items():
        src = binding.get(path)
        if src is None:
            unbound.append(path)
            continue
        if isinstance(src, Tied):
            ignorable.update(src.ignorable)
            if src.path not in specs:
                unbound.append(f"{path} (tied to unknown {src.path})")
            elif tuple(specs[src.path].shape) != tuple(spec.shape):
                wrong.append(f"{path}: tied to {src.path} of shape {list(specs[src.path].shape)}, "
                             f"needs {list(spec.shape)}")
            continue
        try:
            shapes = _piece_shapes(spec, len(src.names))
        except WeightsError as e:
            wrong.append(f"{path}: {e}")
            continue
        ok = True
        for name, shape in zip(src.names, shapes):
            used.add(name)
            if name not in st.entries:
                missing.append(name)
                ok = False
            elif tuple(st.shape(name)) != shape:
                wrong.append(f"{name}: file has {list(st.shape(name))}, config needs {list(shape)}")
                ok = False
            elif spec.role == "table" and st.dtype(name).is_floating_point:
                wrong.append(f"{name}: an integer table is stored as {st.dtype(name)}")
                ok = False
            elif spec.role != "table" and not st.dtype(name).is_floating_point:
                wrong.append(f"{name}: stored as {st.dtype(name)}, needs a floating-point type")
                ok = False
        if ok:
            plan[path] = (spec, src)
    unexpected = sorted(n for n in st.names() if n not in used and n not in ignorable)
    extra_bindings = sorted(p for p in binding if p not in specs)
    if missing or wrong or unexpected or unbound or extra_bindings:
        lines = [f"{st.path}: weights do not fit the configuration"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(sorted(missing)))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes or types ({len(wrong)}): " + "; ".join(wrong))
        if unbound:
            lines.append(f"  parameters the architecture binds to nothing ({len(unbound)}): " + ", ".join(unbound))
        if extra_bindings:
            lines.append(f"  bindings for parameters no part has ({len(extra_bindings)}): " + ", ".join(extra_bindings))
        raise WeightsError("\n".join(lines))

    out: Dict[str, torch.Tensor] = {}
    for path, (spec, src) in plan.items():
        stored = [st.dtype(n) for n in src.names]
        dtype = _target_dtype(spec, stored, compute_dtype)
        parts = [st.tensor(n).to(dtype) for n in src.names]
        t = parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)
        out[path] = t.contiguous().to(device)
    for path, spec in specs.items():
        src = binding.get(path)
        if isinstance(src, Tied):
            out[path] = out[src.path]
    return out


def open_model_weights(model_dir: str) -> SafetensorsFile:
    return SafetensorsFile(os.path.join(model_dir, "model.safetensors"))
