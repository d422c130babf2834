"""Token embedding and the output head.

Embedding: x[i, :] = E[token_i, :], no scaling, no position added
(crates/glassbox-core/src/model.rs:228-231). Head: logits = hs H^T in float32 with H the
embedding when tied (model.rs:190-192, 359-361); no bias, no soft-cap.
"""
from __future__ import annotations

from .. import kernels
from ..weights.binding import ParamSpec
from .base import OutputHead, TokenEmbedding, register_part
from .linear import linear


class Embedding(TokenEmbedding):
    launches_through_kernels_only = True

    def __init__(self, spec=None, *, vocab_size: int, hidden_size: int):
        super().__init__(spec)
        self.vocab_size, self.hidden_size = vocab_size, hidden_size

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size))}

    def forward(self, ctx, tokens, x) -> None:
        kernels.embed(self.params["weight"], tokens, x, ctx.status)


class LmHead(OutputHead):
    launches_through_kernels_only = True

    def __init__(self, spec=None, *, vocab_size: int, hidden_size: int):
        super().__init__(spec)
        self.vocab_size, self.hidden_size = vocab_size, hidden_size

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size))}

    def forward(self, ctx, hs, logits) -> None:
        linear(ctx, hs, self.params["weight"], logits)


register_part("embedding", "embedding", Embedding, replace=True)
register_part("head", "lm_head", LmHead, replace=True)
