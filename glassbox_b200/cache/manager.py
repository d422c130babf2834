"""Host-side bookkeeping of the paged cache: which page holds which tokens of which request.

The device only ever sees block tables and slots; every decision is taken here, on the host, and
can be tested without a GPU.

Layers whose mixers have the same needs (``PagedKvSpec``: kv heads, head size, window) form a
*group* with a page pool and per-request block tables of its own, so a group that keeps only a
window of keys can give pages back early without touching a group that keeps everything. Within a
group one page id addresses the same page in every cache layer of the group, as in Glassbox
where one block id is valid in every layer (crates/glassbox-core/src/kv.rs:17-19, 58-65).

Semantics follow crates/glassbox-core/src/kv.rs: pages of ``page_size`` tokens (16 there, kv.rs:11),
a free stack, reference counts, copy-on-write of a shared partial last page (kv.rs:161-196), fork
(kv.rs:260-266), truncate (kv.rs:237-257), and automatic prefix sharing by a chained FNV-1a hash
of whole pages (kv.rs:45-55, 135-157, 205-233) with unreferenced hashed pages kept for reuse
until space is needed, oldest evicted first (kv.rs:96-110). ``reserve`` is all-or-nothing across
every group. Beside the pages there are *state slots*: one fixed-size slot per live request for
mixers that keep a state instead of keys (and for anything else that is per request and of fixed
size); a slot is handed out at admission, zeroed before first use, copied on fork, and returned
when the request ends.

The bookkeeping itself is C++ (``csrc/host/cache_core.cpp``, loaded with ctypes); this module names
requests by any hashable id, turns return codes into exceptions, and checks the invariants from
outside, on the state the library reports.
"""
from __future__ import annotations

import ctypes
import threading
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from ..csrc import build as _build


class OutOfPages(Exception):
    """Not enough free pages (or no free state slot) for what was asked; nothing was changed."""


@dataclass
class GroupSpec:
    """One cache group as the manager sees it."""
    num_pages: int
    page_size: int = 16
    window: Optional[int] = None
    name: str = ""


_I, _LL, _P = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p
_SIGNATURES = {
    "gbh_cache_new": ([_I, _P, _P, _P, _I, _I, _I], _P),
    "gbh_cache_delete": ([_P], None),
    "gbh_cache_shares_prefixes": ([_P], _I),
    "gbh_cache_add": ([_P, _LL, _P, _I, _P], _I),
    "gbh_cache_reserve": ([_P, _LL, _I, _P, _P], _I),
    "gbh_cache_commit": ([_P, _LL, _P, _I], _I),
    "gbh_cache_commit_many": ([_P, _I, _P, _P, _P], _I),
    "gbh_cache_lengths": ([_P, _I, _P, _P], None),
    "gbh_cache_truncate": ([_P, _LL, _I], _I),
    "gbh_cache_fork": ([_P, _LL, _LL, _P], _I),
    "gbh_cache_free": ([_P, _LL], _I),
    "gbh_cache_has": ([_P, _LL], _I),
    "gbh_cache_length": ([_P, _LL], _I),
    "gbh_cache_slot": ([_P, _LL], _I),
    "gbh_cache_free_pages": ([_P, _I], _I),
    "gbh_cache_ref_count": ([_P, _I, _I], _I),
    "gbh_cache_table": ([_P, _I, _LL, _P, _I], _I),
    "gbh_cache_tokens": ([_P, _LL, _P, _I], _I),
    "gbh_cache_slots": ([_P, _I, _I, _P, _I], _I),
    "gbh_cache_pool": ([_P, _I, _I, _P, _I], _I),
    "gbh_cache_hashes": ([_P, _I, _P, _P, _I, _P], _I),
    "gbh_cache_ids": ([_P, _I, _P, _I], _I),
    "gbh_chain_hash": ([ctypes.c_uint64, _P, _I], ctypes.c_uint64),
    "gbh_plan_step": ([_P, _I, _P, _P, _I, _P, _P, _P, _P, _P, _P, _P], _I),
    "gbh_decode_plan": ([_P, _I, _P, _I, _P, _P, _P], _I),
    "gbh_fill_step": ([_P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _LL, _P, _P, _I, _P, _P, _P], _I),
}
_lib = None
_lock = threading.Lock()


def host_lib():
    """The C++ host library; built at first use."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                handle = ctypes.CDLL(_build.ensure_host_built())
                handle.gbh_last_error.restype = ctypes.c_char_p
                handle.gbh_last_error.argtypes = []
                for name, (args, res) in _SIGNATURES.items():
                    fn = getattr(handle, name)
                    fn.argtypes, fn.restype = args, res
                _lib = handle
    return _lib


def _ints(values, dtype=np.int32) -> np.ndarray:
    return np.ascontiguousarray(values, dtype=dtype)


def chain_hash(prev: int, tokens: Sequence[int]) -> int:
    """FNV-1a over the previous hash and one page of token ids (little-endian u32 bytes),
    crates/glassbox-core/src/kv.rs:45-55."""
    toks = _ints(tokens)
    return int(host_lib().gbh_chain_hash(ctypes.c_uint64(prev), toks.ctypes.data, toks.size))


class _GroupView:
    """What the rest of the engine may know about a group."""

    def __init__(self, spec: GroupSpec):
        self.spec, self.page_size, self.window = spec, spec.page_size, spec.window


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], max_requests: int = 64, share_prefixes: bool = False,
                 has_state: bool = False):
        groups = list(groups)
        for g in groups:
            if g.num_pages <= 0 or g.page_size <= 0:
                raise ValueError("a cache group needs a positive number of pages and a positive page size")
        self._lib = host_lib()
        self.groups = [_GroupView(g) for g in groups]
        self.max_requests = max_requests
        pages, sizes = _ints([g.num_pages for g in groups]), _ints([g.page_size for g in groups])
        windows = _ints([-1 if g.window is None else g.window for g in groups])
        self._h = self._lib.gbh_cache_new(len(groups), pages.ctypes.data, sizes.ctypes.data, windows.ctypes.data,
                                          max_requests, int(share_prefixes), int(has_state))
        if not self._h:
            raise ValueError(self._lib.gbh_last_error().decode())
        # Prefix sharing is only sound when what a page holds is a pure function of the token prefix
        # for every mixer: the library switches it off with windows (pages vanish) or per-request state.
        self.share_prefixes = bool(self._lib.gbh_cache_shares_prefixes(self._h))
        self._ids: Dict[object, int] = {}     # request id -> the 64-bit name the library knows it by
        self._next = 1
        self._scratch = np.empty(3 * max(len(groups), 1) + 2, dtype=np.int32)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and self._lib is not None:
            self._lib.gbh_cache_delete(h)

    def _raise(self, code: int, rid=None):
        msg = self._lib.gbh_last_error().decode()
        if code == 1:
            raise OutOfPages(msg)
        if code == 3:
            raise KeyError(rid)
        raise ValueError(f"request {rid!r}: {msg}" if rid is not None else msg)

    def _id(self, rid) -> int:
        try:
            return self._ids[rid]
        except KeyError:
            raise KeyError(rid) from None

    def native_id(self, rid) -> int:
        """The name under which the library knows the request (for ``fill_step``)."""
        return self._id(rid)

    # ---------------------------------------------------------------------------------- queries
    def has(self, rid) -> bool:
        return rid in self._ids

    def length(self, rid) -> int:
        return self._lib.gbh_cache_length(self._h, self._id(rid))

    def slot_of(self, rid) -> int:
        return self._lib.gbh_cache_slot(self._h, self._id(rid))

    def request_ids(self) -> List[object]:
        return list(self._ids)

    def table(self, group: int, rid) -> List[int]:
        i = self._id(rid)
        n = self._lib.gbh_cache_table(self._h, group, i, None, 0)
        out = np.empty(max(n, 1), dtype=np.int32)
        self._lib.gbh_cache_table(self._h, group, i, out.ctypes.data, n)
        return out[:n].tolist()

    def table_len(self, group: int, rid) -> int:
        return self._lib.gbh_cache_table(self._h, group, self._id(rid), None, 0)

    def tokens(self, rid) -> List[int]:
        i = self._id(rid)
        n = self._lib.gbh_cache_tokens(self._h, i, None, 0)
        out = np.empty(max(n, 1), dtype=np.int32)
        self._lib.gbh_cache_tokens(self._h, i, out.ctypes.data, n)
        return out[:n].tolist()

    def free_pages(self, group: int = 0) -> int:
        return self._lib.gbh_cache_free_pages(self._h, group)

    def used_pages(self, group: int = 0) -> int:
        return self.groups[group].spec.num_pages - self.free_pages(group)

    def num_pages(self, group: int = 0) -> int:
        return self.groups[group].spec.num_pages

    def ref_count(self, group: int, page: int) -> int:
        return self._lib.gbh_cache_ref_count(self._h, group, page)

    def page_hash(self, group: int, page: int) -> Optional[int]:
        """The chained hash under which a full page can be found again, or None."""
        pages = self.groups[group].spec.num_pages
        own = np.empty(pages, dtype=np.uint64)
        self._lib.gbh_cache_hashes(self._h, group, None, None, 0, own.ctypes.data)
        return int(own[page]) if self._pool(group, 3)[page] else None

    def slot(self, group: int, rid, pos: int) -> int:
        """Row of (request, position) in a cache layer of the group (kv.rs:199-201)."""
        ps = self.groups[group].page_size
        page = self.table(group, rid)[pos // ps]
        assert page >= 0, "position lies on a page that was given back"
        return page * ps + pos % ps

    def _slots(self, which: int, drain: bool) -> List[int]:
        out = np.empty(max(self.max_requests, 1), dtype=np.int32)
        n = self._lib.gbh_cache_slots(self._h, which, int(drain), out.ctypes.data, out.size)
        return out[:n].tolist()

    @property
    def free_slots(self) -> List[int]:
        return self._slots(0, False)

    @property
    def fresh_slots(self) -> List[int]:
        return self._slots(1, False)

    def drain_fresh_slots(self) -> List[int]:
        return self._slots(1, True)

    def pages_needed(self, n_tokens: int, group: int = 0) -> int:
        return -(-n_tokens // self.groups[group].page_size)

    # ------------------------------------------------------------------------------ life cycle
    def add_request(self, rid, prompt: Sequence[int] = ()) -> int:
        """Start a request. With prefix sharing, whole leading pages whose token prefix is already
        cached are shared; never the page that holds the last prompt token, which must still run
        to give logits (kv.rs:135-157). Returns the number of tokens already present."""
        if rid in self._ids:
            raise ValueError(f"request {rid!r} exists")
        toks = _ints(prompt)
        present = ctypes.c_int(0)
        i = self._next
        code = self._lib.gbh_cache_add(self._h, i, toks.ctypes.data, toks.size, ctypes.byref(present))
        if code:
            self._raise(code, rid)
        self._next += 1
        self._ids[rid] = i
        return present.value

    def reserve(self, rid, n: int) -> List[Tuple[int, int, int]]:
        """Make room to write positions length .. length+n-1 in every group, all or nothing.
        Returns copy-on-write work as (group, source page, destination page) triples that the
        caller must carry out on the device before the step (kv.rs:161-196)."""
        s = self._scratch
        code = self._lib.gbh_cache_reserve(self._h, self._id(rid), int(n), s.ctypes.data, s[-1:].ctypes.data)
        if code:
            self._raise(code, rid)
        k = int(s[-1])
        return [(int(s[3 * j]), int(s[3 * j + 1]), int(s[3 * j + 2])) for j in range(k)] if k else []

    def commit(self, rid, tokens: Sequence[int]) -> None:
        """Mark ``len(tokens)`` more positions as written; hash pages that became full
        (kv.rs:205-233); give back pages that a window has passed."""
        toks = _ints(tokens)
        code = self._lib.gbh_cache_commit(self._h, self._id(rid), toks.ctypes.data, toks.size)
        if code:
            self._raise(code, rid)

    def commit_many(self, rids, tok_count: np.ndarray, tokens: np.ndarray) -> None:
        """``commit`` for several requests in one call: request e brings ``tok_count[e]`` tokens, flat in
        ``tokens`` (int32)."""
        ids = rids if isinstance(rids, np.ndarray) else np.fromiter((self._id(r) for r in rids), dtype=np.int64, count=len(rids))
        code = self._lib.gbh_cache_commit_many(self._h, len(rids), ids.ctypes.data, tok_count.ctypes.data, tokens.ctypes.data)
        if code:
            self._raise(code)

    def lengths(self, rids) -> np.ndarray:
        """Lengths of several requests (-1 for one that does not exist)."""
        ids = np.fromiter((self._ids.get(r, -1) for r in rids), dtype=np.int64, count=len(rids))
        out = np.empty(max(len(rids), 1), dtype=np.int32)
        self._lib.gbh_cache_lengths(self._h, len(rids), ids.ctypes.data, out.ctypes.data)
        return out[:len(rids)]

    def truncate(self, rid, length: int) -> None:
        """Forget everything after the first ``length`` tokens (kv.rs:237-257). Not available
        once a window has given pages back behind ``length``."""
        code = self._lib.gbh_cache_truncate(self._h, self._id(rid), int(length))
        if code:
            self._raise(code, rid)

    def fork(self, parent, child) -> Tuple[int, int]:
        """New request sharing every page of ``parent`` (kv.rs:260-266). Its state slot is a
        copy, not a share: returns (parent slot, child slot) for the device copy."""
        if child in self._ids:
            raise ValueError(f"request {child!r} exists")
        s = self._scratch
        i = self._next
        code = self._lib.gbh_cache_fork(self._h, self._id(parent), i, s.ctypes.data)
        if code:
            self._raise(code, child)
        self._next += 1
        self._ids[child] = i
        return int(s[0]), int(s[1])

    def free_request(self, rid) -> None:
        """Give back everything the request holds (kv.rs:268-274). Unknown ids are ignored."""
        i = self._ids.pop(rid, None)
        if i is not None:
            self._lib.gbh_cache_free(self._h, i)

    # ------------------------------------------------------------------------------ a scheduler step's plan
    def plan_step(self, rids, remaining, budget: int):
        """Plan one step of continuous batching over the running requests (admission order, with the tokens
        each still has to run) and reserve its pages, in the library (see ``gbh_plan_step``): decoding requests
        first, then prompt portions, under the token budget; when pages run out the most recently admitted
        request is preempted and what it holds given back. Returns (plan as [(index, tokens)], copy-on-write
        triples, number of preempted requests counted from the end of the list, whether a lone request did
        not fit). The caller forgets the preempted requests with ``free_request`` (their pages are gone already)."""
        n = len(rids)
        ids = np.fromiter((self._id(r) for r in rids), dtype=np.int64, count=n)
        rem = _ints(remaining)
        out = np.empty(2 * n + 3 * max(len(self.groups), 1) * max(n, 1) + 4, dtype=np.int32)
        plan_idx, plan_n, copies, tail = out[:n], out[n:2 * n], out[2 * n:-4], out[-4:]
        code = self._lib.gbh_plan_step(self._h, n, ids.ctypes.data, rem.ctypes.data, int(budget), plan_idx.ctypes.data,
                                       plan_n.ctypes.data, tail[0:].ctypes.data, copies.ctypes.data, tail[1:].ctypes.data,
                                       tail[2:].ctypes.data, tail[3:].ctypes.data)
        if code:
            self._raise(code)
        k, nc = int(tail[0]), int(tail[1])
        plan = list(zip(plan_idx[:k].tolist(), plan_n[:k].tolist()))
        triples = [(int(copies[3 * j]), int(copies[3 * j + 1]), int(copies[3 * j + 2])) for j in range(nc)]
        return plan, triples, int(tail[2]), bool(tail[3])

    def native_ids(self, rids) -> np.ndarray:
        """The 64-bit names under which the library knows these requests (for the calls that take them directly)."""
        return np.fromiter((self._ids[r] for r in rids), dtype=np.int64, count=len(rids))

    def decode_plan(self, ids: np.ndarray, max_position: int):
        """Room for one more token of every request named by ``ids`` (native names), all or nothing, in one call (see
        ``gbh_decode_plan``). Returns (code, copy-on-write triples, widest block table): code 0 = reserved; 1 = out of
        pages and 2 = a request is at ``max_position`` (nothing was reserved either way)."""
        n = int(ids.size)
        out = np.empty(3 * max(len(self.groups), 1) * max(n, 1) + 2, dtype=np.int32)
        code = self._lib.gbh_decode_plan(self._h, n, ids.ctypes.data, int(max_position), out.ctypes.data,
                                         out[-2:].ctypes.data, out[-1:].ctypes.data)
        if code:
            return code, [], 0
        nc = int(out[-2])
        return 0, [(int(out[3 * j]), int(out[3 * j + 1]), int(out[3 * j + 2])) for j in range(nc)], int(out[-1])

    # ------------------------------------------------------------------------------ a step's metadata
    def fill_step(self, rids, tok_count: np.ndarray, tokens: np.ndarray, want_count: np.ndarray, want: np.ndarray,
                  n: int, S: int, n_want: int, max_pages: int, offsets: np.ndarray, host: np.ndarray,
                  sample_mask: Optional[np.ndarray] = None, lead: int = 0, pad_after: int = 0,
                  feedback_mask: Optional[np.ndarray] = None):
        """Write the int32 metadata block of a step into ``host`` (see ``gbh_fill_step``): ``pad_after``
        padding sequences follow the first ``lead`` entries, the rest of the padding the last one.
        ``sample_mask`` (uint8, one per wanted row) marks the wanted rows that are sampled from their request's own
        sampling state; ``feedback_mask`` (uint8, one per entry) the single-token entries whose token the device takes from
        what it sampled for the request in the step before. Returns ((start position, slot, first row) per entry as an
        int32 array [E, 3], longest context)."""
        E = len(rids)
        ids = rids if isinstance(rids, np.ndarray) else np.fromiter((self._ids[r] for r in rids), dtype=np.int64, count=E)
        info = np.empty((max(E, 1), 3), dtype=np.int32)
        longest = ctypes.c_int(0)
        k = 0 if sample_mask is None else int(sample_mask.size)
        code = self._lib.gbh_fill_step(
            self._h, E, ids.ctypes.data, tok_count.ctypes.data, tokens.ctypes.data, want_count.ctypes.data,
            want.ctypes.data, int(lead), int(pad_after), n, S, n_want, max_pages, offsets.ctypes.data, host.size,
            host.ctypes.data, sample_mask.ctypes.data if k else None, k,
            feedback_mask.ctypes.data if feedback_mask is not None else None, info.ctypes.data, ctypes.byref(longest))
        if code:
            self._raise(code)
        return info[:E], longest.value

    # ------------------------------------------------------------------------------ invariants
    def _pool(self, group: int, which: int) -> List[int]:
        out = np.empty(self.groups[group].spec.num_pages, dtype=np.int32)
        n = self._lib.gbh_cache_pool(self._h, group, which, out.ctypes.data, out.size)
        return out[:n].tolist()

    def check_invariants(self) -> None:
        """Every page is referenced exactly as often as block tables name it; pages nobody names
        are exactly the free and the cached ones, each once; slots likewise (kv.rs:278-288). Checked
        here, outside the library, on the state it reports."""
        names = set(self._ids.values())
        ids = np.empty(max(len(names), 1) + 8, dtype=np.int64)
        n = self._lib.gbh_cache_ids(self._h, -1, ids.ctypes.data, ids.size)
        assert set(ids[:n].tolist()) == names, "the library's requests and the names given out differ"
        for gi, g in enumerate(self.groups):
            pages = g.spec.num_pages
            refs, free, cached = self._pool(gi, 0), self._pool(gi, 1), self._pool(gi, 2)
            hashed = self._pool(gi, 3)
            want = [0] * pages
            for rid in self._ids:
                for p in self.table(gi, rid):
                    if p >= 0:
                        want[p] += 1
            assert want == refs, f"group {gi}: page reference counts drifted"
            idle = [p for p, r in enumerate(refs) if r == 0]
            pool = free + cached
            assert len(pool) == len(set(pool)), f"group {gi}: a page is on the free lists twice"
            assert sorted(pool) == idle, f"group {gi}: free lists drifted from the reference counts"
            assert all(hashed[p] for p in cached), f"group {gi}: cached page without a hash"
            assert not any(hashed[p] for p in free), f"group {gi}: free page still hashed"
            hs, ps = np.empty(pages, dtype=np.uint64), np.empty(pages, dtype=np.int32)
            own = np.empty(pages, dtype=np.uint64)
            k = self._lib.gbh_cache_hashes(self._h, gi, hs.ctypes.data, ps.ctypes.data, pages, own.ctypes.data)
            assert k <= pages and k == sum(hashed), f"group {gi}: hash index drifted"
            for h, p in zip(hs[:k].tolist(), ps[:k].tolist()):
                assert hashed[p] and int(own[p]) == h, f"group {gi}: hash index drifted"
            n = self._lib.gbh_cache_ids(self._h, gi, ids.ctypes.data, ids.size)
            assert set(ids[:n].tolist()) == names, f"group {gi}: tables and requests differ"
        held = sorted(self.slot_of(r) for r in self._ids)
        assert len(held) == len(set(held)), "a state slot is held twice"
        assert sorted(held + self.free_slots) == list(range(self.max_requests)), "state slots drifted"
