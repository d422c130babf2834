"""A layer: a mixer and a feed-forward wired around the float32 residual stream.

"pre_norm" is x += mixer(norm(x)); x += ffn(norm(x)), with no norms after the parts
(crates/glassbox-core/src/model.rs:251-348). The arrangement is looked up by name, so another
wiring (post-norm, parallel branches) is another registered class.
"""
from __future__ import annotations

from .base import DeferredNorm, Part, build_part, register_part


class PreNormBlock(Part):
    launches_through_kernels_only = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        self.hidden_size = hidden_size
        self.mixer_norm = build_part("norm", spec.mixer_norm, hidden_size=hidden_size)
        self.mixer = build_part("mixer", spec.mixer, hidden_size=hidden_size)
        self.ffn_norm = build_part("norm", spec.ffn_norm, hidden_size=hidden_size)
        self.ffn = build_part("ffn", spec.ffn, hidden_size=hidden_size)

    def sub_parts(self):
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "ffn_norm": self.ffn_norm, "ffn": self.ffn}

    def entry_norm(self):
        """The norm that reads the residual first when this layer runs (whoever runs the layer before may tell
        its last product, through ``ctx.next_norm``, to prepare it)."""
        return self.mixer_norm

    def forward(self, ctx, x, cache, writes_cache: bool, after_mixer=None) -> None:
        """``after_mixer`` (optional) is called once the mixer's kernels are launched: the model uses it
        to let the next layer's mixer start its prefetch beside this layer's feed-forward.
        ``ctx.norm_after_layer`` (optional) is the norm that will read ``x`` after this layer."""
        after_layer = getattr(ctx, "norm_after_layer", None)
        h = DeferredNorm(ctx, self.mixer_norm, x)
        ctx.next_norm = self.ffn_norm          # a hint to the product that adds the mixer's output into x
        self.mixer.forward(ctx, h if self.mixer.accepts_deferred_input else h.tensor(), x, cache, writes_cache)
        if after_mixer is not None:
            after_mixer()
        h = DeferredNorm(ctx, self.ffn_norm, x)
        ctx.next_norm = after_layer
        self.ffn.forward(ctx, h if self.ffn.accepts_deferred_input else h.tensor(), x)
        ctx.next_norm = None


register_part("arrangement", "pre_norm", lambda kind, *, layer_spec, hidden_size: PreNormBlock(layer_spec, hidden_size=hidden_size),
              replace=True)


def build_block(layer_spec, *, hidden_size: int):
    """Build the layer that ``layer_spec.arrangement`` names."""
    return build_part("arrangement", layer_spec.arrangement, layer_spec=layer_spec, hidden_size=hidden_size)
