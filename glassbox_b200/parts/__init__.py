"""The parts a layer is put together from. Importing this package registers the built-in parts."""
from .base import (FeedForward, Mixer, Norm, OutputHead, PagedKvSpec, Part, Position, StateSpec, TokenEmbedding, build_part,
                   register_part, registered)
from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (registration)
from .block import build_block
from .embedding import Embedding, LmHead

__all__ = ["FeedForward", "Mixer", "Norm", "PagedKvSpec", "Part", "Position", "StateSpec", "build_part",
           "register_part", "registered", "build_block", "Embedding", "LmHead", "TokenEmbedding", "OutputHead"]
