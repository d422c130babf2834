"""Typed descriptions of a model: what each layer is made of and in which order layers run.

A ``ModelConfig`` is plain data. It never holds tensors and never knows how a part is
computed; the parts registry (``glassbox_b200.parts``) turns each spec into a part.
Every spec class carries a ``kind`` string, which is the key under which its part class is
registered, so a new mixer / feed-forward / norm / position encoding is a new spec dataclass
plus a new registered part class: nothing in this file changes.

Glassbox reads its sizes off one flat ``Config`` struct inside ``forward``
(crates/glassbox-core/src/model.rs:7-55, 216-226); here the same numbers are split up and
handed to the part that uses them, layer by layer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot describe a runnable model; the message names the key."""


@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding over the first ``rotary_dim`` channels of each head.

    ``pairing`` "half" rotates channel i with channel i + rotary_dim/2 (the Hugging Face
    weight layout, crates/glassbox-core/src/model.rs:110 with interleaved=false).
    """
    theta: float
    rotary_dim: int
    max_position: int
    pairing: str = "half"
    kind: str = "rope"


@dataclass(frozen=True)
class NoPositionSpec:
    kind: str = "none"


@dataclass(frozen=True)
class RmsNormSpec:
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class GqaAttentionSpec:
    """Causal grouped-query attention over a paged key/value cache.

    ``window`` None means every earlier key is visible; an integer w means a query at
    position p sees keys p-w+1 .. p. ``scale`` multiplies the scores before softmax.
    """
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    position: Any
    window: Optional[int] = None
    kind: str = "gqa_attention"


@dataclass(frozen=True)
class SwiGluSpec:
    """Dense gated feed-forward: down(silu(gate(x)) * up(x))."""
    intermediate_size: int
    kind: str = "swiglu"


@dataclass(frozen=True)
class EmbeddingSpec:
    """Token embedding: the float32 residual row of a token is its row of the table, as it is
    (crates/glassbox-core/src/model.rs:228-231). Another kind (a scaled table, a learned position added to it) is
    another registered "embedding" part."""
    kind: str = "embedding"


@dataclass(frozen=True)
class LmHeadSpec:
    """Output head: float32 logits = hidden states times the head matrix, no bias, no cap
    (crates/glassbox-core/src/model.rs:359-361). Another kind is another registered "head" part."""
    kind: str = "lm_head"


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a mixer and a feed-forward, each behind its norm.

    ``arrangement`` names how they are wired around the residual stream; "pre_norm" is
    x += mixer(norm(x)); x += ffn(norm(x)) (crates/glassbox-core/src/model.rs:251-348).
    """
    mixer: Any
    ffn: Any
    mixer_norm: Any
    ffn_norm: Any
    arrangement: str = "pre_norm"


@dataclass(frozen=True)
class RunSpec:
    """One entry of the execution order.

    ``layer`` indexes ``ModelConfig.layers`` (a layer may be named by several entries and
    then runs several times with the same weights). ``cache`` is the cache layer this run
    reads; with ``writes_cache`` False the run writes nothing of its own and reads what an
    earlier run of this step (or of earlier steps) put into that cache layer.
    """
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_position: int
    tie_word_embeddings: bool
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[RunSpec, ...]
    final_norm: Any
    raw: dict = field(default_factory=dict, compare=False, hash=False)
    embedding: Any = EmbeddingSpec()
    head: Any = LmHeadSpec()

    @property
    def num_cache_layers(self) -> int:
        return 1 + max((r.cache for r in self.schedule), default=-1)

    def validate(self) -> None:
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        writers = {}
        for i, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ConfigError(f"schedule[{i}] names layer {run.layer}, but there are {len(self.layers)} layers")
            if run.cache < 0:
                raise ConfigError(f"schedule[{i}] has a negative cache layer")
            if run.writes_cache:
                if run.cache in writers:
                    raise ConfigError(
                        f"schedule[{i}] and schedule[{writers[run.cache]}] both write cache layer {run.cache}")
                writers[run.cache] = i
            elif run.cache not in writers:
                raise ConfigError(f"schedule[{i}] reads cache layer {run.cache} before any run has written it")
        for c in range(self.num_cache_layers):
            if c not in writers:
                raise ConfigError(f"cache layer {c} is never written")
