"""What one step hands to the parts: the rows of the batch, where each row's keys go, and scratch.

Rows are flat: row i is token ``tokens[i]`` of sequence ``row_seq[i]`` (an index into this
step's sequence list) at position ``positions[i]``; rows of one sequence are consecutive and in
order (crates/glassbox-core/src/model.rs:203-215). For every paged cache group the context
carries the block table of each sequence of the step and the cache slot of each row.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..cache.device import DeviceCache, PagedLayerView


@dataclass
class SeqInfo:
    request: object      # the caller's request id
    slot: int            # state slot of the request
    start_pos: int       # position of its first row in this step
    n_rows: int
    first_row: int


class Scratch:
    """Named activation buffers sized for the largest step, reused by every layer."""

    def __init__(self, max_rows: int, dtype: torch.dtype, device):
        self.max_rows, self.dtype, self.device = max_rows, dtype, device
        self._bufs: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}

    def get(self, name: str, shape, dtype: Optional[torch.dtype] = None, grow: bool = False) -> torch.Tensor:
        """A [rows, width] view of the buffer called ``name``. Buffers hold ``max_rows`` rows, except
        with ``grow`` (used for logits, whose row count is the number of wanted rows and whose
        width is the vocabulary): those hold what the largest request so far needed."""
        dtype = dtype or self.dtype
        rows, width = shape
        if rows > self.max_rows:
            raise ValueError(f"a step of {rows} rows exceeds the engine's max_batch_tokens {self.max_rows}")
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.shape[1] < width or buf.shape[0] < rows:
            cap = self.max_rows
            if grow:
                cap = 1
                while cap < rows:
                    cap *= 2
                cap = min(cap, self.max_rows)
            buf = torch.empty((cap, width), dtype=dtype, device=self.device)
            self._bufs[key] = buf
        if buf.shape[1] == width:
            return buf[:rows]
        return buf.view(-1)[:rows * width].view(rows, width)

    def zeros_once(self, name: str, count: int, dtype: torch.dtype) -> torch.Tensor:
        """A flat buffer that is zero when first handed out and is never cleared again: for kernels
        that leave their counters at zero when they finish."""
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < count:
            buf = torch.zeros(count, dtype=dtype, device=self.device)
            self._bufs[key] = buf
        return buf


class WeightOrder:
    """Learns the order in which weight matrices are used in a step (it is the same in every step of
    one model) from the calls themselves, so that a product can ask the memory system for the weights
    of the product two calls further on while it works: parts do not know their neighbours, the
    sequence of calls does."""

    def __init__(self):
        self.following = {}     # data_ptr -> the weight used next
        self._prev = None

    def start_step(self) -> None:
        self._prev = None

    def ahead(self, w: torch.Tensor, distance: int = 2) -> Optional[torch.Tensor]:
        """Record that ``w`` is used now; return the weight expected ``distance`` uses later."""
        if self._prev is not None:
            self.following[self._prev.data_ptr()] = w
        self._prev = w
        t = w
        for _ in range(distance):
            t = self.following.get(t.data_ptr())
            if t is None:
                return None
        return t


class StepContext:
    def __init__(self, *, scratch: Scratch, cache: DeviceCache, status: torch.Tensor, dtype: torch.dtype,
                 grow_scratch: Optional[Scratch] = None):
        self._scratch = scratch
        # Buffers whose size depends on the step (logits, split-attention partials) may be replaced by
        # larger ones later. A context that is recorded into a CUDA graph therefore owns its own set:
        # the graph keeps writing to the addresses it was recorded with.
        self._grow = grow_scratch if grow_scratch is not None else scratch
        self.cache = cache
        self.status = status
        self.dtype = dtype
        self.device = status.device
        self.n = 0
        self.num_wanted = 0
        self.seqs: List[SeqInfo] = []
        self.tokens = self.positions = self.row_seq = self.want_rows = None
        self.seq_first_row = self.seq_start_pos = self.seq_slots = None
        self.group_slots: List[torch.Tensor] = []
        self.group_tables: List[torch.Tensor] = []
        self.max_rows_per_seq = 0
        self.max_context = 0
        self.num_seqs = 0
        self.decode_only = False          # every sequence of the step brings exactly one row
        self.leading_single = 0           # the first this many sequences bring one row each (rows 0 .. this - 1)
        self.token_slots = None           # int32 [rows]: state slot of the rows whose token the device supplies itself, else -1
        self.want_slots = None            # int32 [wanted rows]: state slot of the rows that are sampled from their own state, else -1
        self.weight_order: Optional[WeightOrder] = None
        self.side_stream = None           # a second CUDA stream for work beside the main chain (prefetch)
        self.program = None               # a kernels.Program: decode steps of few rows run as one persistent kernel
        # An RMSNorm may be split between the product that completes the residual rows and the product that reads
        # the normalised rows (parts/linear.py). Whoever wires the parts says which norm comes next:
        self.next_norm = None             # the norm that will read the residual after the product that adds into it next
        self.norm_after_layer = None      # the norm that will read the residual after the layer that runs now
        self.prepared_norm = None         # parts.base.PreparedNorm: what the last such product left for that norm

    def scratch(self, name: str, shape, dtype: Optional[torch.dtype] = None, grow: bool = False) -> torch.Tensor:
        return (self._grow if grow else self._scratch).get(name, shape, dtype, grow)

    def zeros_once(self, name: str, count: int, dtype: torch.dtype) -> torch.Tensor:
        return self._scratch.zeros_once(name, count, dtype)

    @property
    def max_rows(self) -> int:
        return self._scratch.max_rows

    def cache_view(self, cache_layer: int):
        view = self.cache.layer_view(cache_layer)
        if isinstance(view, PagedLayerView):
            view.slots = self.group_slots[view.group]
            view.block_tables = self.group_tables[view.group]
        return view
