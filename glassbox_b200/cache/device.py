"""Device storage behind the cache manager: page pools for the paged groups and slot arrays for
fixed-size per-request state. This file allocates and hands out views; it decides nothing.

Paged group storage: K and V each ``[cache layers of the group, pages, kv_heads, page_size,
head_dim]`` in the activation dtype, so one (page, kv head) is a contiguous
``page_size x head_dim`` tile, which is what the attention kernels stream.
State storage: one tensor ``[max_requests, *shape]`` per cache layer whose mixer asked for it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..parts.base import PagedKvSpec, StateSpec


@dataclass
class PagedLayerView:
    """What a mixer sees of its cache layer during one step."""
    k: torch.Tensor                 # [pages, kv_heads, page_size, head_dim]
    v: torch.Tensor
    page_size: int
    group: int
    slots: Optional[torch.Tensor] = None          # int32 [n]: row -> page*page_size + offset
    block_tables: Optional[torch.Tensor] = None   # int32 [sequences of the step, max pages]


@dataclass
class StateLayerView:
    state: torch.Tensor             # [max_requests, *shape]; index with ctx.seq_slots


class DeviceCache:
    def __init__(self, layer_specs: List[object], pages_per_group, page_size: int, max_requests: int,
                 dtype: torch.dtype, device):
        """``layer_specs[c]`` is the cache spec of cache layer ``c`` (PagedKvSpec, StateSpec or
        None). ``pages_per_group(spec) -> int`` sizes each group's pool."""
        self.page_size = page_size
        self.max_requests = max_requests
        self.group_specs: List[PagedKvSpec] = []
        self.group_of_layer: Dict[int, int] = {}
        self.index_in_group: Dict[int, int] = {}
        members: List[List[int]] = []
        self.state: Dict[int, torch.Tensor] = {}
        for c, spec in enumerate(layer_specs):
            if isinstance(spec, PagedKvSpec):
                if spec not in self.group_specs:
                    self.group_specs.append(spec)
                    members.append([])
                g = self.group_specs.index(spec)
                self.group_of_layer[c] = g
                self.index_in_group[c] = len(members[g])
                members[g].append(c)
            elif isinstance(spec, StateSpec):
                self.state[c] = torch.zeros((max_requests,) + tuple(spec.shape), dtype=spec.dtype, device=device)
            elif spec is not None:
                raise TypeError(f"cache layer {c}: unknown cache spec {spec!r}")
        # Sampling state of each live request, in its state slot: {generator state low word, high word, temperature
        # bits, unused}; zero (greedy) for a fresh slot, copied on fork like every other per-request state.
        self.sampling = torch.zeros((max_requests, 4), dtype=torch.int32, device=device)
        # The token the sampling kernel chose last for the request in each slot: the next step can take it from here on
        # the device, before the host has read it.
        self.last_token = torch.zeros(max_requests, dtype=torch.int32, device=device)
        self.group_pages = [int(pages_per_group(s)) for s in self.group_specs]
        self.k: List[torch.Tensor] = []
        self.v: List[torch.Tensor] = []
        for g, spec in enumerate(self.group_specs):
            shape = (len(members[g]), self.group_pages[g], spec.num_kv_heads, page_size, spec.head_dim)
            self.k.append(torch.zeros(shape, dtype=dtype, device=device))
            self.v.append(torch.zeros(shape, dtype=dtype, device=device))

    @property
    def has_state(self) -> bool:
        return bool(self.state)

    def bytes_per_token(self) -> int:
        total = 0
        for g, spec in enumerate(self.group_specs):
            total += 2 * self.k[g].shape[0] * spec.num_kv_heads * spec.head_dim * self.k[g].element_size()
        return total

    def layer_view(self, cache_layer: int):
        if cache_layer in self.group_of_layer:
            g = self.group_of_layer[cache_layer]
            i = self.index_in_group[cache_layer]
            return PagedLayerView(k=self.k[g][i], v=self.v[g][i], page_size=self.page_size, group=g)
        if cache_layer in self.state:
            return StateLayerView(state=self.state[cache_layer])
        return None

    def zero_slots(self, slots: List[int]) -> None:
        """Fresh slots start from zero: the mixers' states, and the sampling state (temperature 0: greedy)."""
        if slots:
            idx = torch.tensor(slots, dtype=torch.long, device=self.sampling.device)
            self.sampling.index_fill_(0, idx, 0)
            for t in self.state.values():
                t.index_fill_(0, idx, 0)

    def copy_slot(self, src: int, dst: int) -> None:
        for t in self.state.values():
            t[dst].copy_(t[src])
        self.sampling[dst].copy_(self.sampling[src])
        self.last_token[dst].copy_(self.last_token[src])

    def set_sampling(self, slot: int, temperature: float, rng_state: int) -> None:
        import struct
        bits = struct.unpack("<i", struct.pack("<f", float(temperature)))[0]
        lo, hi = rng_state & 0xFFFFFFFF, (rng_state >> 32) & 0xFFFFFFFF
        as_i32 = lambda u: u - (1 << 32) if u >= (1 << 31) else u
        row = torch.tensor([as_i32(lo), as_i32(hi), bits, 0], dtype=torch.int32)
        self.sampling[slot].copy_(row, non_blocking=False)

    def get_rng_state(self, slot: int) -> int:
        lo, hi = (int(v) & 0xFFFFFFFF for v in self.sampling[slot, :2].tolist())
        return (hi << 32) | lo
