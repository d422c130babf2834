"""The engine: a loaded model, its cache, and the one step function.

``Engine.step(entries)`` runs one batch of (request, its next tokens): portions of prompts beside
single decoded tokens, cut anywhere. It runs only the rows it is given, reads everything earlier
from the cache, and returns float32 logits at the wanted places. It is the counterpart of
``Model::forward`` in crates/glassbox-core/src/model.rs:207-362 together with the
reserve/commit calls its callers make around it (crates/glassbox-core/src/lib.rs:39-50).
Trace replay, the scheduler and the generator all drive this same function.
"""
from __future__ import annotations

import gc
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
from .context import Scratch, SeqInfo, StepContext, WeightOrder
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
                 config: Optional[ModelConfig] = None, use_graphs: bool = True, use_programs: bool = False,
                 group_pages=None):
        """``cache_tokens`` / ``num_pages`` size the page pool of every cache group alike; ``group_pages`` (a function
        from a group's ``PagedKvSpec`` to a number of pages) sizes each group on its own, for models whose groups need
        different amounts: a group that keeps a window of keys needs far fewer pages than one that keeps them all."""
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
        pages_for = group_pages if group_pages is not None else (lambda spec: self.num_pages)
        self.device_cache = DeviceCache(layer_specs, pages_for, self.page_size, self.max_requests, self.dtype, self.device)
        groups = [GroupSpec(num_pages=self.device_cache.group_pages[i], page_size=self.page_size, window=s.window,
                            name=f"group{i}") for i, s in enumerate(self.device_cache.group_specs)]
        self.cache = CacheManager(groups, max_requests=self.max_requests, share_prefixes=share_prefixes,
                                  has_state=self.device_cache.has_state)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        # a step recorded as a graph runs at a rounded shape: a few rows more than the tokens it brings
        self._scratch_rows = self.max_batch_tokens + self.max_requests + 128
        self.scratch = Scratch(self._scratch_rows, self.dtype, self.device)
        self.ctx = StepContext(scratch=self.scratch, cache=self.device_cache, status=self.status, dtype=self.dtype)
        self.weight_order = WeightOrder()
        self.ctx.weight_order = self.weight_order
        self.side_stream = torch.cuda.Stream(device=self.device)
        self.ctx.side_stream = self.side_stream
        self.use_programs = bool(use_programs) and self.dtype == torch.bfloat16 and self.model.program_safe
        if self.use_programs:
            self.ctx.program = kernels.Program()
        self._meta_dev = torch.empty(1 << 16, dtype=torch.int32, device=self.device)
        self._stage = [torch.empty(1 << 16, dtype=torch.int32).pin_memory() for _ in range(4)]
        self._stage_np = [t.numpy() for t in self._stage]
        self._stage_events = [None] * len(self._stage)
        self._stage_next = 0
        self.steps = 0
        self.use_graphs = bool(use_graphs)
        self.max_graph_batch = 64
        self._graphs: Dict[tuple, dict] = {}
        self._layouts: Dict[tuple, dict] = {}
        self._seen: Dict[tuple, int] = {}
        self.max_graphs = 128
        self.graph_replays = 0
        self.sampled: Optional[torch.Tensor] = None
        self._sampled_host: Optional[torch.Tensor] = None
        self._ones = np.ones(self.max_graph_batch, dtype=np.int32)
        self._zeros = np.zeros(self.max_graph_batch, dtype=np.int32)
        self._ones_u8 = np.ones(self.max_graph_batch, dtype=np.uint8)
        # sampled tokens of launched decode steps land in pinned buffers that take turns (two steps may be in flight)
        self._decode_out = [(torch.empty(self.max_graph_batch, dtype=torch.int32).pin_memory(), torch.cuda.Event())
                            for _ in range(3)]
        self._decode_turn = 0
        self.h2d_bytes_last = 0

    # ---------------------------------------------------------------------------- requests
    def add_request(self, request, prompt: Sequence[int] = ()) -> int:
        """Admit a request; returns how many leading prompt tokens are already cached. Its state slot starts from zero
        (mixers' states; greedy sampling until ``set_sampling`` says otherwise)."""
        reused = self.cache.add_request(request, prompt)
        self.device_cache.zero_slots(self.cache.drain_fresh_slots())
        return reused

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
        self.run_copies(self.cache.reserve(request, n))

    def run_copies(self, copies) -> None:
        """Carry out copy-on-write work, (group, source page, destination page) triples, on the device."""
        if copies:
            by_group: Dict[int, List[List[int]]] = {}
            for g, src, dst in copies:
                by_group.setdefault(g, []).append([src, dst])
            for g, pairs in by_group.items():
                t = torch.tensor(pairs, dtype=torch.int32, device=self.device)
                kernels.copy_pages(self.device_cache.k[g], self.device_cache.v[g], t)

    # ----------------------------------------------------------------------- step metadata
    def _stage_buffer(self, size: int) -> np.ndarray:
        """The next pinned staging buffer of the ring as a numpy array of ``size`` int32 (a ring, so that a
        buffer is not rewritten while its copy may still be in flight)."""
        if size > self._stage[0].numel():
            cap = 1 << int(size - 1).bit_length()
            self._stage = [torch.empty(cap, dtype=torch.int32).pin_memory() for _ in range(len(self._stage))]
            self._stage_np = [t.numpy() for t in self._stage]
            self._stage_events = [None] * len(self._stage)
        i = self._stage_next = (self._stage_next + 1) % len(self._stage)
        if self._stage_events[i] is not None:
            self._stage_events[i].synchronize()
        return self._stage_np[i][:size]

    def _stage_copy(self, host: np.ndarray, dev: torch.Tensor) -> None:
        """One host-to-device copy of the step's metadata; ``host`` is the array ``_stage_buffer`` gave last."""
        i, n = self._stage_next, host.size
        dev[:n].copy_(self._stage[i][:n], non_blocking=True)
        if self._stage_events[i] is None:
            self._stage_events[i] = torch.cuda.Event()
        self._stage_events[i].record()
        self.h2d_bytes_last = n * 4

    def _layout(self, n: int, S: int, n_want: int, max_pages: int):
        key = (n, S, n_want, max_pages)
        off = self._layouts.get(key)
        if off is not None:
            return off
        if len(self._layouts) > 4096:
            self._layouts.clear()
        off, cur = {}, 0
        for name, size in (("tokens", n), ("positions", n), ("row_seq", n), ("want", n_want),
                           ("seq_first_row", S + 1), ("seq_start_pos", S), ("seq_slots", S), ("want_slots", n_want),
                           ("token_slots", n)):
            off[name] = cur
            cur += size
        for g in range(len(self.cache.groups)):
            off[f"slots{g}"] = cur
            cur += n
            off[f"tables{g}"] = cur
            cur += S * max_pages
        off["_size"] = cur
        names = ["tokens", "positions", "row_seq", "want", "seq_first_row", "seq_start_pos", "seq_slots", "want_slots",
                 "token_slots"] + \
            [f"{kind}{g}" for g in range(len(self.cache.groups)) for kind in ("slots", "tables")]
        off["_array"] = np.array([off[k] for k in names], dtype=np.int64)   # the order the host library reads
        self._layouts[key] = off
        return off

    def _fill(self, entries, off, n, S, n_want, max_pages, sampling=None, lead=0, pad_after=0) -> np.ndarray:
        """Host copy of the metadata block, written by the C++ host library from the cache manager's
        tables. Rows and sequences beyond the entries (a batch padded to a fixed shape) get position
        -1, slot -1 and empty tables: every kernel skips them."""
        E = len(entries)
        tok_count = np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=E)
        want_count = np.fromiter((len(e.want) for e in entries), dtype=np.int32, count=E)
        if int(tok_count.sum()) == E:
            tokens = np.fromiter((e.tokens[0] for e in entries), dtype=np.int32, count=E)
        else:
            tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries]).astype(np.int32)
        want = np.fromiter((w for e in entries for w in e.want), dtype=np.int32, count=int(want_count.sum()))
        self._tok_count, self._tokens = tok_count, tokens      # kept for the commit that follows the step
        host = self._stage_buffer(off["_size"])
        mask = None
        if sampling is not None:
            mask = np.ascontiguousarray(sampling, dtype=np.uint8)
            if mask.size != int(want_count.sum()):
                raise ValueError(f"sampling names {mask.size} rows, the step wants {int(want_count.sum())}")
        info, self._max_ctx = self.cache.fill_step([e.request for e in entries], tok_count, tokens, want_count, want,
                                                   n, S, n_want, max_pages, off["_array"], host, mask, lead, pad_after)
        self._seqs = [SeqInfo(request=e.request, slot=int(info[i, 1]), start_pos=int(info[i, 0]), n_rows=int(tok_count[i]),
                              first_row=int(info[i, 2])) for i, e in enumerate(entries)]
        return host

    def _bind(self, ctx: StepContext, dev: torch.Tensor, off, n, S, n_want, max_pages) -> None:
        n_groups = len(self.cache.groups)
        ctx.n, ctx.num_wanted = n, n_want
        ctx.tokens = dev[off["tokens"]:off["tokens"] + n]
        ctx.positions = dev[off["positions"]:off["positions"] + n]
        ctx.row_seq = dev[off["row_seq"]:off["row_seq"] + n]
        ctx.want_rows = dev[off["want"]:off["want"] + n_want]
        ctx.seq_first_row = dev[off["seq_first_row"]:off["seq_first_row"] + S + 1]
        ctx.seq_start_pos = dev[off["seq_start_pos"]:off["seq_start_pos"] + S]
        ctx.seq_slots = dev[off["seq_slots"]:off["seq_slots"] + S]
        ctx.want_slots = dev[off["want_slots"]:off["want_slots"] + n_want]
        ctx.token_slots = dev[off["token_slots"]:off["token_slots"] + n]
        ctx.group_slots = [dev[off[f"slots{g}"]:off[f"slots{g}"] + n] for g in range(n_groups)]
        ctx.group_tables = [dev[off[f"tables{g}"]:off[f"tables{g}"] + S * max_pages].view(S, max_pages)
                            for g in range(n_groups)]
        ctx.num_seqs = S

    def _validate(self, entries) -> int:
        cfg = self.config
        n = sum(len(e.tokens) for e in entries)
        if n == 0:
            raise ValueError("a step needs at least one token")
        if n > self.max_batch_tokens:
            raise ValueError(f"a step of {n} tokens exceeds max_batch_tokens {self.max_batch_tokens}")
        if len({e.request for e in entries}) != len(entries):
            raise ValueError("a request appears twice in one step")
        lengths = self.cache.lengths([e.request for e in entries])
        for e, have in zip(entries, lengths):
            k = len(e.tokens)
            if have < 0:
                raise KeyError(f"unknown request {e.request!r}; add_request first")
            if not k:
                raise ValueError(f"request {e.request!r} brings no tokens")
            if have + k > cfg.max_position:
                raise ValueError(f"request {e.request!r} would reach {have + k} tokens, beyond max_position "
                                 f"{cfg.max_position}")
            for w in e.want:
                if not 0 <= w < k:
                    raise ValueError(f"request {e.request!r}: wanted index {w} outside its {k} tokens")
        return n

    def step(self, entries: Sequence[StepEntry], reserve: bool = True, commit: bool = True,
             sampling=None) -> torch.Tensor:
        """Run one batch. Returns float32 logits ``[total wanted, vocab]`` on the device, in the
        order of the entries and of each entry's ``want``; the tensor is scratch that the next
        step overwrites. With ``reserve`` True room is reserved for every entry first, all or nothing:
        on ``OutOfPages`` no request holds more pages than before. With ``reserve`` False the caller has
        already reserved room for every entry (the scheduler does, to decide about preemption first). With ``sampling`` (one
        flag per wanted row) the sampling kernel runs in the same step and ``self.sampled`` holds the chosen token of
        each wanted row (int32, on the device): rows whose flag is set are drawn from their request's own sampling
        state (``set_sampling``: temperature and random generator, kept in the request's state slot on the device and
        advanced there), the others are the row's greedy choice.

        A step made only of single decoded tokens runs as a CUDA graph of fixed shape (batch and
        table sizes rounded up to powers of two, padding rows skipped by every kernel); any other
        step launches its kernels one by one. Both run the same kernels on the same data."""
        n = self._validate(entries)
        self.sampled = None
        if reserve:
            done = []
            try:
                for e in entries:
                    self.reserve(e.request, len(e.tokens))
                    done.append(e.request)
            except OutOfPages:
                # all or nothing: the pages that earlier entries of this step were given go back (a page copied
                # for a write stays with its request: it holds the same keys as the page it was copied from)
                for rid in done:
                    self.cache.truncate(rid, self.cache.length(rid))
                raise
        self.device_cache.zero_slots(self.cache.drain_fresh_slots())
        n_groups = len(self.cache.groups)
        S = len(entries)
        max_pages = max(max(self.cache.table_len(g, e.request) for e in entries) for g in range(n_groups)) \
            if n_groups else 1
        n_want = sum(len(e.want) for e in entries)
        decode_only = self.use_graphs and n == S and n_want == S and S <= self.max_graph_batch \
            and self.model.recordable(True)
        if decode_only:
            logits = self._step_graph(entries, S, max_pages, sampling)
        else:
            logits = None
            max_rows = max(len(e.tokens) for e in entries)
            lead = 0                      # single-token requests at the head of the batch (the scheduler's order)
            while lead < S and len(entries[lead].tokens) == 1:
                lead += 1
            small_logits = (n_want + 8) * self.config.vocab_size * 4 <= (64 << 20)   # each graph owns its logits buffer
            if self.use_graphs and small_logits and self.model.recordable(n == S):
                # A step is replayed as a CUDA graph of a rounded shape, so that batches which differ a little share
                # one: the single-token requests at its head counted in eights (padding sequences behind them), the
                # other requests in powers of two, the rows in 64s, the wanted rows in eights, the table width in
                # powers of two (the flash kernel's grid covers the longest run such a shape can hold). A shape is recorded the second time it is seen: a
                # portioned prompt repeats its shape, and so does a service that fills its token budget.
                Pb = max(8, 1 << max(max_pages - 1, 0).bit_length())
                lead_b = -(-lead // 8) * 8
                rest = S - lead
                rest_b = 1 << max(rest - 1, 0).bit_length() if rest else 0
                S_b = lead_b + rest_b
                n_b = lead_b + -(-(n - lead + rest_b - rest) // 64) * 64
                want_b = -(-n_want // 8) * 8
                tiles = -(-(n_b - lead_b) // 128)      # the most row tiles a request of this shape can have
                key = ("step", n_b, lead_b, rest_b, want_b, Pb)
                g = self._graphs.get(key)
                off = self._layout(n_b, S_b, want_b, Pb)
                if g is None:
                    if len(self._seen) > 4096:
                        self._seen.clear()
                    self._seen[key] = self._seen.get(key, 0) + 1
                    if self._seen[key] >= 2 and len(self._graphs) < self.max_graphs:
                        host = self._fill(entries, off, n_b, S_b, want_b, Pb, sampling, lead, lead_b - lead)
                        g = self._capture(key, off, host, n_b, S_b, want_b, Pb, tiles * 128, decode_only=(rest == 0),
                                          lead=lead_b)
                        self.sampled = g["sampled"][:n_want] if sampling is not None else None
                        logits = g["logits"][:n_want]       # the warm-up run of the capture computed this step
                else:
                    host = self._fill(entries, off, n_b, S_b, want_b, Pb, sampling, lead, lead_b - lead)
                    self._stage_copy(host, g["meta"])
                    g["graph"].replay()
                    kernels.launch_count += g["nodes"]
                    self.graph_replays += 1
                    self.sampled = g["sampled"][:n_want] if sampling is not None else None
                    logits = g["logits"][:n_want]
            if logits is None:
                off = self._layout(n, S, n_want, max_pages)
                host = self._fill(entries, off, n, S, n_want, max_pages, sampling)
                if off["_size"] > self._meta_dev.numel():
                    self._meta_dev = torch.empty(1 << int(off["_size"] - 1).bit_length(), dtype=torch.int32,
                                                 device=self.device)
                self._stage_copy(host, self._meta_dev)
                ctx = self.ctx
                self._bind(ctx, self._meta_dev, off, n, S, n_want, max_pages)
                ctx.seqs, ctx.max_context = self._seqs, self._max_ctx
                ctx.max_rows_per_seq = max_rows
                ctx.decode_only = (n == S)
                ctx.leading_single = lead
                logits = self.model.forward(ctx)
                if sampling is not None and n_want:
                    self.sampled = self.scratch.get("sampled", (n_want, 1), torch.int32, grow=True).view(-1)
                    kernels.sample(logits, self.sampled, want_slots=ctx.want_slots, state=self.device_cache.sampling,
                                   last_token=self.device_cache.last_token)
        if commit:
            self.cache.commit_many([e.request for e in entries], self._tok_count, self._tokens)
        self.steps += 1
        return logits

    def _decode_graph(self, Sb: int, Pb: int):
        """The CUDA graph of a decode step of ``Sb`` rows with block tables ``Pb`` wide, recorded if new."""
        key = (Sb, Pb)
        g = self._graphs.get(key)
        if g is None:
            off = self._layout(Sb, Sb, Sb, Pb)
            seqs, longest = getattr(self, "_seqs", None), getattr(self, "_max_ctx", 0)
            blank = self._fill([], off, Sb, Sb, Sb, Pb)          # an all-padding batch: every row skipped
            self._seqs, self._max_ctx = seqs, longest
            g = self._capture(key, off, blank, Sb, Sb, Sb, Pb, 1, decode_only=True)
        return g

    def warm_up(self, max_batch: int, max_context: int) -> int:
        """Record the decode graphs a service will need before it needs them: every batch bucket (powers of
        two up to ``max_batch``) at every table width (powers of two up to ``max_context`` tokens). Recording
        a graph takes tens of milliseconds; without this it happens inside the first step of each new shape,
        also when a batch shrinks because requests end. Returns the number of graphs recorded."""
        if not self.use_graphs or not self.model.recordable(True):
            return 0
        before = len(self._graphs)
        max_pages = -(-min(int(max_context), self.config.max_position) // self.page_size)
        Pb = 8
        widths = []
        while True:
            widths.append(Pb)
            if Pb >= max_pages:
                break
            Pb *= 2
        Sb = 1
        while Sb <= min(int(max_batch), self.max_graph_batch):
            for Pb in widths:
                if len(self._graphs) >= self.max_graphs:
                    return len(self._graphs) - before
                self._decode_graph(Sb, Pb)
            Sb *= 2
        return len(self._graphs) - before

    def _step_graph(self, entries, S: int, max_pages: int, sampling) -> torch.Tensor:
        Sb = 1 << max(S - 1, 0).bit_length()
        Pb = max(8, 1 << max(max_pages - 1, 0).bit_length())
        off = self._layout(Sb, Sb, Sb, Pb)
        g = self._decode_graph(Sb, Pb)          # (may fill a blank batch of its own: before this step's metadata)
        host = self._fill(entries, off, Sb, Sb, Sb, Pb, sampling)
        self._stage_copy(host, g["meta"])
        g["graph"].replay()
        kernels.launch_count += g["nodes"]
        self.sampled = g["sampled"][:S]
        self.graph_replays += 1
        return g["logits"][:S]

    def decode_launch(self, requests, tokens: Optional[np.ndarray], sample_mask: np.ndarray):
        """Launch the steady state of generation in as few host operations as it takes, and do not wait for it: every
        request of ``requests`` brings one token and wants its next token, sampled on the device (from the request's own
        sampling state where ``sample_mask[i]`` is set, else greedily). ``tokens`` (int32) are the tokens they bring;
        None says that each request's token is the one the device sampled for it in the step before, which the host
        need not have read yet: the step takes it from the device, and the cache learns the token values later
        (``decode_commit_tokens``). One native call plans the step (room for one token each, all or nothing), one fills
        the metadata block, one sends it, launches the step's recorded graph and fetches the sampled tokens.

        Returns a handle for ``decode_wait``, or None when this path does not take the step as it stands (no graphs,
        too many requests, a request at ``max_position``, pages run out): nothing has changed then."""
        n = len(requests)
        if not (self.use_graphs and 0 < n <= self.max_graph_batch and self.model.recordable(True)):
            return None
        cache = self.cache
        ids = cache.native_ids(requests)
        code, copies, max_pages = cache.decode_plan(ids, self.config.max_position)
        if code:
            return None
        self.run_copies(copies)
        Sb = 1 << max(n - 1, 0).bit_length()
        Pb = max(8, 1 << max(max_pages - 1, 0).bit_length())
        off = self._layout(Sb, Sb, Sb, Pb)
        g = self._decode_graph(Sb, Pb)
        ones, zeros = self._ones[:n], self._zeros[:n]
        host = self._stage_buffer(off["_size"])
        self._stage_events[self._stage_next] = None      # (every such step is waited for before the ring comes round)
        fed = tokens is None
        cache.fill_step(ids, ones, zeros if fed else tokens, ones, zeros, Sb, Sb, Sb, Pb, off["_array"], host, sample_mask,
                        feedback_mask=self._ones_u8[:n] if fed else None)
        turn = self._decode_turn = (self._decode_turn + 1) % len(self._decode_out)
        out, event = self._decode_out[turn]
        kernels.step_io(host.ctypes.data, g["meta"], off["_size"] * 4, g["exec"], g["sampled"], out, n, g["nodes"])
        event.record()
        self.h2d_bytes_last = off["_size"] * 4
        if not fed:
            cache.commit_many(ids, ones, tokens)         # host bookkeeping, while the device works
        self.graph_replays += 1
        self.steps += 1
        self.sampled = None
        return {"ids": ids, "n": n, "out": out, "event": event, "fed": fed}

    def decode_wait(self, handle) -> np.ndarray:
        """The sampled tokens of a launched decode step (int32 numpy array, valid until two more steps are launched)."""
        handle["event"].synchronize()
        return handle["out"].numpy()[:handle["n"]]

    def decode_commit_tokens(self, handle, tokens: np.ndarray) -> None:
        """Tell the cache which tokens a launched step that took them from the device was given (the host knows them
        now): one per request of the step, in its order."""
        if handle["fed"]:
            self.cache.commit_many(handle["ids"], self._ones[:handle["n"]], np.ascontiguousarray(tokens, dtype=np.int32))
            handle["fed"] = False

    def decode_fast(self, requests, tokens: np.ndarray, sample_mask: np.ndarray):
        """``decode_launch`` and ``decode_wait`` in one: the sampled tokens, or None if the path declines the step."""
        handle = self.decode_launch(requests, tokens, sample_mask)
        return None if handle is None else self.decode_wait(handle)

    def _capture(self, key, off, host, n, S, n_want, Pb, max_rows, decode_only, lead=0):
        """Record the kernels of one step shape into a CUDA graph with a metadata block, logits and
        scratch of its own. The kernels run once outside capture first, on the metadata given (for a
        decode shape an all-padding batch; otherwise the real step, which is thereby computed), so
        that every scratch buffer exists; then they are recorded."""
        meta = torch.empty(off["_size"], dtype=torch.int32, device=self.device)
        ctx = StepContext(scratch=self.scratch, cache=self.device_cache, status=self.status, dtype=self.dtype,
                          grow_scratch=Scratch(self._scratch_rows, self.dtype, self.device))
        self._bind(ctx, meta, off, n, S, n_want, Pb)
        ctx.weight_order = self.weight_order
        ctx.side_stream = self.side_stream
        if self.use_programs:
            ctx.program = kernels.Program()
        ctx.seqs = [SeqInfo(request=None, slot=0, start_pos=0, n_rows=1, first_row=i) for i in range(S)]
        # (the longest context a step of this shape can hold: what its block tables cover)
        ctx.max_context = min(self.config.max_position, Pb * self.page_size)
        ctx.max_rows_per_seq, ctx.decode_only = max_rows, decode_only
        ctx.leading_single = lead
        meta.copy_(torch.from_numpy(host))
        sampled = torch.zeros(max(n_want, 1), dtype=torch.int32, device=self.device)

        def run():
            if decode_only and S == n:      # rows whose token is what the step before sampled take it on the device
                kernels.resolve_tokens(ctx.tokens, ctx.token_slots, self.device_cache.last_token)
            logits = self.model.forward(ctx)
            kernels.sample(logits, sampled[:n_want], want_slots=ctx.want_slots, state=self.device_cache.sampling,
                           last_token=self.device_cache.last_token)
            return logits

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            run()                                            # warm-up: allocates scratch
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = kernels.launch_count
        # Nothing may free device memory while the stream records: an engine that was dropped earlier and is
        # collected now would destroy its own graphs and their memory pools in the middle of this recording,
        # which invalidates it. So what is garbage is collected first and the collector rests meanwhile.
        was_enabled = gc.isenabled()
        gc.collect()
        gc.disable()
        try:
            with torch.cuda.graph(graph):
                logits = run()
        finally:
            if was_enabled:
                gc.enable()
        g = {"graph": graph, "meta": meta, "logits": logits, "sampled": sampled, "ctx": ctx,
             "nodes": kernels.launch_count - before, "exec": int(graph.raw_cuda_graph_exec())}
        self._graphs[key] = g
        return g

    @property
    def max_position(self) -> int:
        return self.config.max_position

    def set_sampling(self, request, temperature: float, rng_state: int) -> None:
        """Put a request's sampling state into its state slot on the device: the temperature (0: greedy) and the state
        of its xorshift64* generator. From then on ``step(..., sampling=...)`` draws the request's tokens on the device
        and advances the generator there; a fork copies the state with the slot."""
        self.device_cache.set_sampling(self.cache.slot_of(request), temperature, rng_state)

    def rng_state(self, request) -> int:
        """The state of the request's random generator as the device has advanced it (synchronises)."""
        return self.device_cache.get_rng_state(self.cache.slot_of(request))

    def rng_state_of_slot(self, slot: int) -> int:
        """... by slot number: what the slot's last holder left (a slot keeps its contents until it is given out again)."""
        return self.device_cache.get_rng_state(slot)

    def sample(self, logits: torch.Tensor, rows: Sequence[int], samplers, contexts) -> List[int]:
        """Next token for ``logits[rows[i]]`` under ``samplers[i]``. Greedy and plain temperature sampling were done
        by the device kernel inside the step (``step(..., sampling=...)``, from the request's own state slot) and are
        only read here; requests with further filters are sampled on the host from a copy of their row."""
        w = logits.shape[0]
        if self.sampled is None or self.sampled.shape[0] != w:
            self.sampled = self.scratch.get("sampled", (w, 1), torch.int32, grow=True).view(-1)
            kernels.sample(logits, self.sampled)
        if self._sampled_host is None or self._sampled_host.numel() < w:
            self._sampled_host = torch.empty(max(w, 64), dtype=torch.int32).pin_memory()
        self._sampled_host[:w].copy_(self.sampled, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        picked = self._sampled_host.numpy()
        self.sampled = None
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
