"""The Llama-family dense decoder as Glassbox runs it (SmolLM2): RMSNorm, half-split RoPE,
grouped-query attention, SwiGLU, tied or untied LM head, no biases
(crates/glassbox-core/src/model.rs:57-79, 207-362).

This file only *describes* the architecture: which config.json keys it reads and how its
safetensors names map onto part parameters. The math lives in the parts.
"""
from __future__ import annotations

import math
import struct

from ..config.registry import Architecture, register_architecture
from ..config.specs import (ConfigError, GqaAttentionSpec, LayerSpec, ModelConfig, RmsNormSpec, RopeSpec,
                            RunSpec, SwiGluSpec)
from ..weights.binding import Stacked, Tied

NAME = "LlamaForCausalLM"

_REQUIRED = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
             "num_key_value_heads", "vocab_size")


def _positive_int(raw: dict, key: str) -> int:
    v = raw[key]
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: '{key}' must be a positive integer, got {v!r}")
    return v


def _as_f32(x: float) -> float:
    """Round to the nearest float32, as a Rust ``f32`` field does on parse."""
    return struct.unpack("<f", struct.pack("<f", float(x)))[0]


def parse_llama_config(raw: dict) -> ModelConfig:
    """Read exactly the keys Glassbox reads, with its defaults
    (crates/glassbox-core/src/model.rs:7-55): the six sizes are required; ``rms_norm_eps``
    defaults to 1e-5, ``rope_theta`` to 10000 (also looked up under ``rope_parameters``),
    ``tie_word_embeddings`` to false, ``head_dim`` to hidden/heads and
    ``max_position_embeddings`` to 2048. Unknown keys are ignored. Unlike Glassbox, sizes
    that cannot work together are refused here instead of failing later.
    """
    missing = [k for k in _REQUIRED if k not in raw]
    if missing:
        raise ConfigError(f"config.json: missing required key(s): {', '.join(missing)}")
    d = _positive_int(raw, "hidden_size")
    inter = _positive_int(raw, "intermediate_size")
    n_layers = _positive_int(raw, "num_hidden_layers")
    nh = _positive_int(raw, "num_attention_heads")
    nkv = _positive_int(raw, "num_key_value_heads")
    vocab = _positive_int(raw, "vocab_size")
    if raw.get("head_dim") is not None:
        hd = _positive_int(raw, "head_dim")
    else:
        if d % nh:
            raise ConfigError(f"config.json: hidden_size {d} is not divisible by num_attention_heads {nh} "
                              "and no 'head_dim' is given")
        hd = d // nh
    if nh % nkv:
        raise ConfigError(f"config.json: num_attention_heads {nh} is not a multiple of num_key_value_heads {nkv}")
    if hd % 2:
        raise ConfigError(f"config.json: head_dim {hd} must be even for rotary position encoding")
    eps = raw.get("rms_norm_eps", 1e-5)
    if not isinstance(eps, (int, float)) or isinstance(eps, bool) or not eps > 0:
        raise ConfigError(f"config.json: 'rms_norm_eps' must be a positive number, got {eps!r}")
    theta = raw.get("rope_theta")
    if theta is None:
        nested = raw.get("rope_parameters")
        theta = nested.get("rope_theta") if isinstance(nested, dict) else None
    if theta is None:
        theta = 10000.0
    if not isinstance(theta, (int, float)) or isinstance(theta, bool) or not theta > 0:
        raise ConfigError(f"config.json: 'rope_theta' must be a positive number, got {theta!r}")
    tie = raw.get("tie_word_embeddings", False)
    if not isinstance(tie, bool):
        raise ConfigError(f"config.json: 'tie_word_embeddings' must be true or false, got {tie!r}")
    max_pos = raw["max_position_embeddings"] if "max_position_embeddings" in raw else 2048
    if isinstance(max_pos, bool) or not isinstance(max_pos, int) or max_pos <= 0:
        raise ConfigError(f"config.json: 'max_position_embeddings' must be a positive integer, got {max_pos!r}")

    eps = _as_f32(eps)
    norm = RmsNormSpec(eps=eps)
    rope = RopeSpec(theta=_as_f32(theta), rotary_dim=hd, max_position=max_pos, pairing="half")
    attn = GqaAttentionSpec(num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                            scale=_as_f32(1.0 / _as_f32(math.sqrt(hd))), position=rope, window=None)
    layer = LayerSpec(mixer=attn, ffn=SwiGluSpec(intermediate_size=inter), mixer_norm=norm, ffn_norm=norm,
                      arrangement="pre_norm")
    return ModelConfig(
        architecture=NAME, vocab_size=vocab, hidden_size=d, max_position=max_pos, tie_word_embeddings=tie,
        layers=tuple(layer for _ in range(n_layers)),
        schedule=tuple(RunSpec(layer=i, cache=i) for i in range(n_layers)),
        final_norm=norm, raw=dict(raw))


def bind_llama_weights(config: ModelConfig) -> dict:
    """Hugging Face tensor names for each part parameter (crates/glassbox-core/src/load.rs:50-78).
    Q, K, V rows are stacked into one matrix and so are gate and up rows (load.rs:55-65). The
    head reuses the embedding when the config ties them; an untied config must bring
    ``lm_head.weight`` (Glassbox would tie silently, load.rs:70-75: here that is an error).
    """
    b = {"embed.weight": Stacked(("model.embed_tokens.weight",)),
         "final_norm.weight": Stacked(("model.norm.weight",))}
    for i in range(len(config.layers)):
        p = f"model.layers.{i}"
        b[f"layers.{i}.mixer_norm.weight"] = Stacked((f"{p}.input_layernorm.weight",))
        b[f"layers.{i}.mixer.wqkv"] = Stacked((f"{p}.self_attn.q_proj.weight", f"{p}.self_attn.k_proj.weight",
                                               f"{p}.self_attn.v_proj.weight"))
        b[f"layers.{i}.mixer.wo"] = Stacked((f"{p}.self_attn.o_proj.weight",))
        b[f"layers.{i}.ffn_norm.weight"] = Stacked((f"{p}.post_attention_layernorm.weight",))
        b[f"layers.{i}.ffn.w_gate_up"] = Stacked((f"{p}.mlp.gate_proj.weight", f"{p}.mlp.up_proj.weight"))
        b[f"layers.{i}.ffn.w_down"] = Stacked((f"{p}.mlp.down_proj.weight",))
    if config.tie_word_embeddings:
        b["head.weight"] = Tied("embed.weight", ignorable=("lm_head.weight",))
    else:
        b["head.weight"] = Stacked(("lm_head.weight",))
    return b


def make_llama_raw_config(*, hidden_size, intermediate_size, num_hidden_layers, num_attention_heads,
                          num_key_value_heads, vocab_size, head_dim=None, rope_theta=10000.0, rms_norm_eps=1e-5,
                          tie_word_embeddings=False, max_position_embeddings=2048) -> dict:
    raw = {
        "architectures": [NAME], "model_type": "llama", "hidden_size": hidden_size,
        "intermediate_size": intermediate_size, "num_hidden_layers": num_hidden_layers,
        "num_attention_heads": num_attention_heads, "num_key_value_heads": num_key_value_heads,
        "vocab_size": vocab_size, "rope_theta": rope_theta, "rms_norm_eps": rms_norm_eps,
        "tie_word_embeddings": tie_word_embeddings, "max_position_embeddings": max_position_embeddings,
        "hidden_act": "silu",
    }
    if head_dim is not None:
        raw["head_dim"] = head_dim
    return raw


register_architecture(Architecture(name=NAME, parse=parse_llama_config, bind=bind_llama_weights,
                                   make_raw_config=make_llama_raw_config), replace=True)
