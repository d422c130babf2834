"""Typed model configuration and the architecture registry."""
from .specs import (ConfigError, GqaAttentionSpec, LayerSpec, ModelConfig, NoPositionSpec, RmsNormSpec,
                    RopeSpec, RunSpec, SwiGluSpec)
from .registry import (Architecture, architecture_names, get_architecture, load_config, parse_config,
                       register_architecture)

__all__ = [
    "ConfigError", "GqaAttentionSpec", "LayerSpec", "ModelConfig", "NoPositionSpec", "RmsNormSpec", "RopeSpec",
    "RunSpec", "SwiGluSpec", "Architecture", "architecture_names", "get_architecture", "load_config",
    "parse_config", "register_architecture",
]
