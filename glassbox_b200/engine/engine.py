"""The engine: a loaded model, its cache, and the one step function.

``Engine.step(entries)`` runs one batch of (request, its next tokens): portions of prompts beside
single decoded tokens, cut anywhere. It runs only the rows it is given, reads everything earlier
from the cache, and returns float32 logits at the wanted places. It is the counterpart of
``Model::forward`` in crates/glassbox-core/src/model.rs:207-362 together with the
reserve/commit calls its callers make around it (crates/glassbox-core/src/lib.rs:39-50).
Trace replay, the scheduler and the generator all drive this same function.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import kernels
from ..cache.device import DeviceCache
from ..cache.manager import CacheManager, GroupSpec, OutOfPages
from ..config.registry import get_architecture, load_config
from ..config.specs import ModelConfig
from ..weights.loader import load_parameters, open_model_weights
from .context import Scratch, SeqInfo, StepContext
from .model import DecoderModel

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"unsupported compute dtype {name}")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"unknown dtype {name!r}; use bfloat16 or float32") from None


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens, and the indices among them whose logits
    are wanted (possibly none)."""
    request: object
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)


class Engine:
    def __init__(self, model_dir: str, dtype="bfloat16", *, cache_tokens: Optional[int] = None,
                 num_pages: Optional[int] = None, page_size: int = 16, max_batch_tokens: int = 2048,
                 max_requests: int = 64, share_prefixes: bool = False, device: str = "cuda:0",
                 config: Optional[ModelConfig] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("glassbox_b200 needs a CUDA device: every kernel is CUDA and there is no CPU path")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        kernels.lib()  # build/load now, so a missing toolchain fails here and loudly
        self.dtype = parse_dtype(dtype)
        self.config = config if config is not None else load_config(model_dir)
        self.model = DecoderModel(self.config)
        arch = get_architecture(self.config.architecture)
        with open_model_weights(model_dir) as st:
            params = load_parameters(self.model.param_specs(), arch.bind(self.config), st, self.dtype, self.device)
        self.model.bind(params)
        self.page_size = int(page_size)
        if num_pages is None:
            tokens = cache_tokens if cache_tokens is not None else self.config.max_position
            num_pages = -(-int(tokens) // self.page_size)
        self.num_pages = int(num_pages)
        self.max_batch_tokens = int(max_batch_tokens)
        self.max_requests = int(max_requests)
        layer_specs = self.model.cache_layer_specs()
        self.device_cache = DeviceCache(layer_specs, lambda spec: self.num_pages, self.page_size, self.max_requests,
                                        self.dtype, self.device)
        groups = [GroupSpec(num_pages=self.num_pages, page_size=self.page_size, window=s.window, name=f"group{i}")
                  for i, s in enumerate(self.device_cache.group_specs)]
        self.cache = CacheManager(groups, max_requests=self.max_requests, share_prefixes=share_prefixes,
                                  has_state=self.device_cache.has_state)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.scratch = Scratch(self.max_batch_tokens, self.dtype, self.device)
        self.ctx = StepContext(scratch=self.scratch, cache=self.device_cache, status=self.status, dtype=self.dtype)
        self._meta_dev = torch.empty(1 << 16, dtype=torch.int32, device=self.device)
        self._stage = [torch.empty(1 << 16, dtype=torch.int32).pin_memory() for _ in range(4)]
        self._stage_events = [None] * len(self._stage)
        self._stage_next = 0
        self.steps = 0

    # ---------------------------------------------------------------------------- requests
    def add_request(self, request, prompt: Sequence[int] = ()) -> int:
        """Admit a request; returns how many leading prompt tokens are already cached."""
        return self.cache.add_request(request, prompt)

    def free_request(self, request) -> None:
        self.cache.free_request(request)

    def fork(self, parent, child) -> None:
        src, dst = self.cache.fork(parent, child)
        self.device_cache.copy_slot(src, dst)

    def length(self, request) -> int:
        return self.cache.length(request)

    # -------------------------------------------------------------------------------- step
    def reserve(self, request, n: int) -> None:
        """Make room for ``n`` more tokens of ``request`` (raises ``OutOfPages``; nothing changes
        then) and carry out any copy-on-write on the device."""
        copies = self.cache.reserve(request, n)
        if copies:
            by_group: Dict[int, List[List[int]]] = {}
            for g, src, dst in copies:
                by_group.setdefault(g, []).append([src, dst])
            for g, pairs in by_group.items():
                t = torch.tensor(pairs, dtype=torch.int32, device=self.device)
                kernels.copy_pages(self.device_cache.k[g], self.device_cache.v[g], t)

    def _upload(self, host: np.ndarray) -> torch.Tensor:
        n = host.size
        if n > self._meta_dev.numel():
            cap = 1 << int(n - 1).bit_length()
            self._meta_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._stage = [torch.empty(cap, dtype=torch.int32).pin_memory() for _ in range(len(self._stage))]
            self._stage_events = [None] * len(self._stage)
        i = self._stage_next
        self._stage_next = (i + 1) % len(self._stage)
        if self._stage_events[i] is not None:
            self._stage_events[i].synchronize()
        stage = self._stage[i]
        stage.numpy()[:n] = host
        self._meta_dev[:n].copy_(stage[:n], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._stage_events[i] = ev
        self.h2d_bytes_last = n * 4
        return self._meta_dev

    def step(self, entries: Sequence[StepEntry], reserve: bool = True, commit: bool = True) -> torch.Tensor:
        """Run one batch. Returns float32 logits ``[total wanted, vocab]`` on the device, in the
        order of the entries and of each entry's ``want``; the tensor is scratch that the next
        step overwrites. With ``reserve`` False the caller has already reserved room for every
        entry (the scheduler does, to decide about preemption first)."""
        cfg = self.config
        ps = self.page_size
        n_groups = len(self.cache.groups)
        n = sum(len(e.tokens) for e in entries)
        if n == 0:
            raise ValueError("a step needs at least one token")
        if n > self.max_batch_tokens:
            raise ValueError(f"a step of {n} tokens exceeds max_batch_tokens {self.max_batch_tokens}")
        seen = set()
        for e in entries:
            if not self.cache.has(e.request):
                raise KeyError(f"unknown request {e.request!r}; add_request first")
            if e.request in seen:
                raise ValueError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            if not len(e.tokens):
                raise ValueError(f"request {e.request!r} brings no tokens")
            end = self.cache.length(e.request) + len(e.tokens)
            if end > cfg.max_position:
                raise ValueError(f"request {e.request!r} would reach {end} tokens, beyond max_position "
                                 f"{cfg.max_position}")
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise ValueError(f"request {e.request!r}: wanted index {w} outside its {len(e.tokens)} tokens")
        if reserve:
            for e in entries:
                self.reserve(e.request, len(e.tokens))
        self.device_cache.zero_slots(self.cache.drain_fresh_slots())

        S = len(entries)
        max_pages = max(max(len(self.cache.table(g, e.request)) for e in entries) for g in range(n_groups)) \
            if n_groups else 1
        n_want = sum(len(e.want) for e in entries)
        # layout of the int32 metadata block
        off = {}
        cur = 0
        for name, size in (("tokens", n), ("positions", n), ("row_seq", n), ("want", n_want),
                           ("seq_first_row", S + 1), ("seq_start_pos", S), ("seq_slots", S)):
            off[name] = cur
            cur += size
        for g in range(n_groups):
            off[f"slots{g}"] = cur
            cur += n
            off[f"tables{g}"] = cur
            cur += S * max_pages
        host = np.empty(cur, dtype=np.int32)
        seqs: List[SeqInfo] = []
        row = 0
        wi = off["want"]
        max_ctx = 0
        for si, e in enumerate(entries):
            k = len(e.tokens)
            start = self.cache.length(e.request)
            seqs.append(SeqInfo(request=e.request, slot=self.cache.slot_of(e.request), start_pos=start, n_rows=k,
                                first_row=row))
            host[off["tokens"] + row:off["tokens"] + row + k] = np.asarray(e.tokens, dtype=np.int64).astype(np.int32)
            pos = np.arange(start, start + k, dtype=np.int32)
            host[off["positions"] + row:off["positions"] + row + k] = pos
            host[off["row_seq"] + row:off["row_seq"] + row + k] = si
            for w in e.want:
                host[wi] = row + w
                wi += 1
            host[off["seq_first_row"] + si] = row
            host[off["seq_start_pos"] + si] = start
            host[off["seq_slots"] + si] = seqs[-1].slot
            for g in range(n_groups):
                table = np.asarray(self.cache.table(g, e.request), dtype=np.int32)
                t0 = off[f"tables{g}"] + si * max_pages
                host[t0:t0 + max_pages] = -1
                host[t0:t0 + table.size] = table
                host[off[f"slots{g}"] + row:off[f"slots{g}"] + row + k] = table[pos // ps] * ps + pos % ps
            row += k
            max_ctx = max(max_ctx, start + k)
        host[off["seq_first_row"] + S] = row
        dev = self._upload(host)

        ctx = self.ctx
        ctx.n, ctx.num_wanted, ctx.seqs = n, n_want, seqs
        ctx.tokens = dev[off["tokens"]:off["tokens"] + n]
        ctx.positions = dev[off["positions"]:off["positions"] + n]
        ctx.row_seq = dev[off["row_seq"]:off["row_seq"] + n]
        ctx.want_rows = dev[off["want"]:off["want"] + n_want]
        ctx.seq_first_row = dev[off["seq_first_row"]:off["seq_first_row"] + S + 1]
        ctx.seq_start_pos = dev[off["seq_start_pos"]:off["seq_start_pos"] + S]
        ctx.seq_slots = dev[off["seq_slots"]:off["seq_slots"] + S]
        ctx.group_slots = [dev[off[f"slots{g}"]:off[f"slots{g}"] + n] for g in range(n_groups)]
        ctx.group_tables = [dev[off[f"tables{g}"]:off[f"tables{g}"] + S * max_pages].view(S, max_pages)
                            for g in range(n_groups)]
        ctx.max_rows_per_seq = max(s.n_rows for s in seqs)
        ctx.max_context = max_ctx

        logits = self.model.forward(ctx)
        if commit:
            for e in entries:
                self.cache.commit(e.request, e.tokens)
        self.steps += 1
        return logits

    @property
    def max_position(self) -> int:
        return self.config.max_position

    def sample(self, logits: torch.Tensor, rows: Sequence[int], samplers, contexts) -> List[int]:
        """Next token for ``logits[rows[i]]`` under ``samplers[i]``. Greedy and plain temperature
        sampling run in the device kernel (the random number comes from the request's own
        generator); requests with further filters are sampled on the host from a copy of the row."""
        w = logits.shape[0]
        temps = np.zeros(w, dtype=np.float32)
        unif = np.zeros(w, dtype=np.float32)
        host_rows = []
        for r, s in zip(rows, samplers):
            if s.config.needs_host:
                host_rows.append(r)
            elif not s.config.greedy:
                temps[r] = s.config.temperature
                unif[r] = s.uniform()
        params = torch.from_numpy(np.stack([temps, unif])).to(self.device, non_blocking=True)
        out = self.scratch.get("sampled", (w, 1), torch.int32, grow=True).view(-1)
        kernels.sample(logits, out, params[0], params[1])
        picked = out.cpu().numpy()
        result = []
        for r, s, ctx_tokens in zip(rows, samplers, contexts):
            if s.config.needs_host:
                result.append(s.sample(logits[r].cpu().numpy(), ctx_tokens))
            else:
                result.append(int(picked[r]))
        return result

    def check(self) -> None:
        """Synchronise and raise if any kernel since the last check skipped a bad index."""
        kernels.check_status(self.status)

    # ------------------------------------------------------------------------------ figures
    def weight_bytes(self) -> int:
        return self.model.weight_bytes()

    def cache_bytes_per_token(self) -> int:
        return self.device_cache.bytes_per_token()
