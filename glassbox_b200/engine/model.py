"""The one model class: an embedding, layers built from parts, an execution order, a final norm
and a head, every one of them a registered part named by the configuration. Which architecture it is
shows only in its ``ModelConfig``.

Forward order follows crates/glassbox-core/src/model.rs:207-362: embed every row, run the layers
(here: the entries of ``config.schedule``), then final norm and head on the wanted rows only.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels
from ..config.specs import ModelConfig
from ..parts import build_block, build_part
from ..parts.base import Mixer, Part
from ..weights.binding import ParamSpec


def _all_parts(part: Part):
    yield part
    for sub in part.sub_parts().values():
        yield from _all_parts(sub)


def _collect(prefix: str, part: Part, out: Dict[str, ParamSpec], owners: Dict[str, tuple]) -> None:
    for name, spec in part.param_specs().items():
        out[f"{prefix}.{name}"] = spec
        owners[f"{prefix}.{name}"] = (part, name)
    for sub_name, sub in part.sub_parts().items():
        _collect(f"{prefix}.{sub_name}", sub, out, owners)


class DecoderModel:
    def __init__(self, config: ModelConfig):
        config.validate()
        self.config = config
        d = config.hidden_size
        self.embed = build_part("embedding", config.embedding, vocab_size=config.vocab_size, hidden_size=d)
        self.layers = [build_block(spec, hidden_size=d) for spec in config.layers]
        self.final_norm = build_part("norm", config.final_norm, hidden_size=d)
        self.head = build_part("head", config.head, vocab_size=config.vocab_size, hidden_size=d)
        self._owners: Dict[str, tuple] = {}
        self._specs: Dict[str, ParamSpec] = {}
        _collect("embed", self.embed, self._specs, self._owners)
        for i, layer in enumerate(self.layers):
            _collect(f"layers.{i}", layer, self._specs, self._owners)
        _collect("final_norm", self.final_norm, self._specs, self._owners)
        _collect("head", self.head, self._specs, self._owners)
        #: whether a decode step of this model may be recorded as a program for the persistent kernel: only when
        #: no part enqueues device work behind the kernel library's back
        self.program_safe = all(p.launches_through_kernels_only for p in self.parts())

    def param_specs(self) -> Dict[str, ParamSpec]:
        return dict(self._specs)

    def parts(self):
        for top in (self.embed, *self.layers, self.final_norm, self.head):
            yield from _all_parts(top)

    def recordable(self, decode_only: bool) -> bool:
        """Whether every part lets a step of this kind be replayed as a CUDA graph (see ``Part.recordable``)."""
        return all(p.recordable(decode_only) for p in self.parts())

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        grouped: Dict[int, tuple] = {}
        for path, tensor in params.items():
            part, name = self._owners[path]
            grouped.setdefault(id(part), (part, {}))[1][name] = tensor
        for part, named in grouped.values():
            part.bind(named)
        self.params = dict(params)

    def cache_layer_specs(self) -> List[object]:
        """The cache spec of each cache layer: that of the mixer of the run that writes it."""
        specs: List[object] = [None] * self.config.num_cache_layers
        for run in self.config.schedule:
            mixer = getattr(self.layers[run.layer], "mixer", None)
            spec = mixer.cache_spec() if mixer is not None else None
            if run.writes_cache:
                specs[run.cache] = spec
        for run in self.config.schedule:
            if not run.writes_cache:
                mixer = getattr(self.layers[run.layer], "mixer", None)
                spec = mixer.cache_spec() if mixer is not None else None
                if spec != specs[run.cache]:
                    raise ValueError(f"a run of layer {run.layer} reads cache layer {run.cache}, whose writer keeps "
                                     f"{specs[run.cache]!r}, but needs {spec!r}")
        return specs

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for t in self.params.values():
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    def forward(self, ctx) -> torch.Tensor:
        """Run the rows of ``ctx`` through the model; returns float32 logits [wanted rows, vocab]."""
        n, d = ctx.n, self.config.hidden_size
        if getattr(ctx, "weight_order", None) is not None:
            ctx.weight_order.start_step()
        x = ctx.scratch("x", (n, d), torch.float32)
        program = getattr(ctx, "program", None)
        if program is not None and not (ctx.decode_only and self.program_safe and program.takes_rows(n)):
            program = None
        if program is not None:
            kernels.program_begin(program, ctx.status)
        try:
            return self._forward(ctx, x, program is not None)
        finally:
            if program is not None:
                kernels.program_end()

    def _forward(self, ctx, x, in_program: bool) -> torch.Tensor:
        n, d = ctx.n, self.config.hidden_size
        ctx.next_norm = ctx.norm_after_layer = ctx.prepared_norm = None
        self.embed.forward(ctx, ctx.tokens, x)
        schedule = self.config.schedule
        # (a program's persistent kernel asks for the next layer's keys and values itself)
        side = ctx.side_stream if ctx.decode_only and not in_program else None
        pending = False
        for i, run in enumerate(schedule):
            hook = None
            if side is not None and i + 1 < len(schedule):
                nxt = schedule[i + 1]
                mixer = getattr(self.layers[nxt.layer], "mixer", None)
                if mixer is not None and type(mixer).prefetch is not Mixer.prefetch:
                    def hook(mixer=mixer, cache_layer=nxt.cache):
                        # beside this layer's feed-forward, on a second stream: the next mixer's prefetch
                        main = torch.cuda.current_stream()
                        side.wait_stream(main)
                        with torch.cuda.stream(side):
                            mixer.prefetch(ctx, ctx.cache_view(cache_layer))
            if pending:
                torch.cuda.current_stream().wait_stream(side)   # the prefetch kernel must not outlive the step
                pending = False
            # which norm reads x after this layer: the next layer's first one, if it says which that is
            entry = getattr(self.layers[schedule[i + 1].layer], "entry_norm", None) if i + 1 < len(schedule) else None
            ctx.norm_after_layer = entry() if entry is not None else None
            self.layers[run.layer].forward(ctx, x, ctx.cache_view(run.cache), run.writes_cache, after_mixer=hook) \
                if hook is not None else self.layers[run.layer].forward(ctx, x, ctx.cache_view(run.cache), run.writes_cache)
            pending = hook is not None
        if pending:
            torch.cuda.current_stream().wait_stream(side)
        ctx.norm_after_layer = None
        w = ctx.num_wanted
        logits = ctx.scratch("logits", (w, self.config.vocab_size), torch.float32, grow=True)
        if w:
            hs = ctx.scratch("hs", (w, d))
            self.final_norm.forward(ctx, x, hs, rows=ctx.want_rows)
            self.head.forward(ctx, hs, logits)
        return logits
