"""Typed model configuration and the architecture registry."""
from .specs import (ConfigError, EmbeddingSpec, GqaAttentionSpec, LayerSpec, LmHeadSpec, ModelConfig, NoPositionSpec,
                    RmsNormSpec, RopeSpec, RunSpec, SwiGluSpec)
from .registry import (Architecture, architecture_names, get_architecture, load_config, parse_config,
                       register_architecture)

__all__ = [
    "ConfigError", "EmbeddingSpec", "LmHeadSpec", "GqaAttentionSpec", "LayerSpec", "ModelConfig", "NoPositionSpec", "RmsNormSpec", "RopeSpec",
    "RunSpec", "SwiGluSpec", "Architecture", "architecture_names", "get_architecture", "load_config",
    "parse_config", "register_architecture",
]
