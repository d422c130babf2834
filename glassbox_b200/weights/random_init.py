"""Random-weights mode: write a model folder (config.json, model.safetensors) from a raw
configuration and a seed, so that tests and benchmarks go through the same loader as real
checkpoints.

Matrices are N(0, 0.02); gains are 1 + N(0, 0.01), away from exactly one "so a mistake in
applying them shows up" (tools/reference/make_standin.py:90-94). Glassbox's own
``Model::random`` (crates/glassbox-core/src/model.rs:124-161) draws uniform weights with
unit gains and is always tied; the untied case matters here, so the head follows the config.

Each file tensor is drawn from its own generator seeded by (seed, tensor name), so the values
do not depend on the order in which tensors are produced.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict

import torch

from ..config.registry import parse_config
from .binding import Stacked, Tied
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
GAIN_STD = 0.01


def _generator(seed: int, name: str) -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(digest[:8], "little") & ((1 << 63) - 1))
    return g


def random_tensors(raw_config: dict, seed: int, store_dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """File tensors (by their safetensors names) for ``raw_config``."""
    from ..config.registry import get_architecture
    from ..engine.model import DecoderModel
    config = parse_config(raw_config)
    arch = get_architecture(config.architecture)
    model = DecoderModel(config)
    specs = model.param_specs()
    binding = arch.bind(config)
    out: Dict[str, torch.Tensor] = {}
    for path, spec in specs.items():
        src = binding[path]
        if isinstance(src, Tied):
            continue
        assert isinstance(src, Stacked)
        rows = spec.pieces if len(src.names) > 1 else (spec.shape[0],)
        for name, r in zip(src.names, rows):
            shape = (r,) + tuple(spec.shape[1:])
            g = _generator(seed, name)
            if spec.role == "gain":
                t = 1.0 + GAIN_STD * torch.randn(shape, generator=g, dtype=torch.float32)
            elif spec.role == "table":
                t = torch.randint(0, 2 ** 15, shape, generator=g, dtype=torch.int32)
            else:
                t = MATRIX_STD * torch.randn(shape, generator=g, dtype=torch.float32)
            out[name] = t if spec.role == "table" else t.to(store_dtype)
    return out


def write_random_model(model_dir: str, raw_config: dict, seed: int,
                       store_dtype: torch.dtype = torch.bfloat16) -> str:
    """Create ``model_dir`` with config.json and model.safetensors; returns ``model_dir``."""
    os.makedirs(model_dir, exist_ok=True)
    tensors = random_tensors(raw_config, seed, store_dtype)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(raw_config, f, indent=1, sort_keys=True)
        f.write("\n")
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "glassbox_b200_random_seed": str(seed)})
    return model_dir
