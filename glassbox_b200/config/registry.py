"""One registry from an architecture's name (config.json ``architectures[0]``) to its model.

An ``Architecture`` is two functions and nothing else: ``parse`` turns the architecture's own
config.json keys into a ``ModelConfig`` (the typed, per-layer description), and ``bind`` says
which safetensors tensor names feed which parameter of which part. The model object itself is
always the generic ``glassbox_b200.engine.model.DecoderModel`` assembled from parts, so adding
an architecture never touches the step function, the cache, the scheduler or the kernels.

Glassbox has no registry: its loader always builds the Llama ``Model``
(crates/glassbox-server/src/main.rs:44-64). The registry is this engine's addition.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, List

from .specs import ConfigError, ModelConfig


@dataclass(frozen=True)
class Architecture:
    name: str
    #: raw config.json dict -> ModelConfig
    parse: Callable[[dict], ModelConfig]
    #: ModelConfig -> {parameter path: weight source}; see glassbox_b200.weights.binding
    bind: Callable[[ModelConfig], dict]
    #: (keyword sizes) -> raw config.json dict, used by the random-weights mode and tests
    make_raw_config: Callable[..., dict] = None


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {arch.name!r} is already registered")
    _ARCHITECTURES[arch.name] = arch


def architecture_names() -> List[str]:
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {', '.join(architecture_names()) or '(none)'}") from None


def parse_config(raw: dict) -> ModelConfig:
    """Pick the architecture by ``architectures[0]`` and let it read its own keys."""
    archs = raw.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    config = get_architecture(archs[0]).parse(raw)
    config.validate()
    return config


def load_config(model_dir: str) -> ModelConfig:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return parse_config(raw)
