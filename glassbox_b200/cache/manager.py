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
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple


class OutOfPages(Exception):
    """Not enough free pages (or no free state slot) for what was asked; nothing was changed."""


_FNV_OFFSET = 0xCBF29CE484222325
_FNV_PRIME = 0x100000001B3
_MASK = (1 << 64) - 1


def chain_hash(prev: int, tokens: Sequence[int]) -> int:
    """FNV-1a over the previous hash and one page of token ids (little-endian u32 bytes),
    crates/glassbox-core/src/kv.rs:45-55."""
    h = (prev ^ _FNV_OFFSET) & _MASK
    for t in tokens:
        for b in int(t).to_bytes(4, "little"):
            h ^= b
            h = (h * _FNV_PRIME) & _MASK
    return h


@dataclass
class GroupSpec:
    """One cache group as the manager sees it."""
    num_pages: int
    page_size: int = 16
    window: Optional[int] = None
    name: str = ""


class _Group:
    def __init__(self, spec: GroupSpec, share_prefixes: bool):
        if spec.num_pages <= 0 or spec.page_size <= 0:
            raise ValueError("a cache group needs a positive number of pages and a positive page size")
        self.spec = spec
        self.page_size = spec.page_size
        self.window = spec.window
        self.refs = [0] * spec.num_pages
        # Page 0 pops first (kv.rs:67).
        self.free: List[int] = list(range(spec.num_pages - 1, -1, -1))
        self.tables: Dict[object, List[int]] = {}
        self.share = share_prefixes and spec.window is None
        self.by_hash: Dict[int, int] = {}
        self.page_hash: List[Optional[int]] = [None] * spec.num_pages
        self.cached: List[int] = []  # unreferenced pages kept for prefix reuse, oldest first

    # -- pool ------------------------------------------------------------------------------
    def free_pages(self) -> int:
        return len(self.free) + len(self.cached)

    def alloc(self) -> int:
        if self.free:
            p = self.free.pop()
        elif self.cached:
            p = self.cached.pop(0)
            h = self.page_hash[p]
            if h is not None:
                self.page_hash[p] = None
                self.by_hash.pop(h, None)
        else:
            raise OutOfPages()
        assert self.refs[p] == 0, "allocated a page that is still referenced"
        self.refs[p] = 1
        return p

    def release(self, p: int) -> None:
        assert self.refs[p] > 0, f"page {p} freed twice"
        self.refs[p] -= 1
        if self.refs[p] == 0:
            if self.page_hash[p] is not None:
                self.cached.append(p)
            else:
                self.free.append(p)

    def retain(self, p: int) -> None:
        if self.refs[p] == 0:
            self.cached.remove(p)
        self.refs[p] += 1

    # -- what a reservation needs --------------------------------------------------------------
    def first_live_page(self, length: int) -> int:
        """Index of the first page a query at position >= ``length`` can still see."""
        if self.window is None:
            return 0
        return max(0, length - self.window + 1) // self.page_size

    def plan(self, table: List[int], length: int, n: int) -> Tuple[int, bool]:
        """(new pages, copy-on-write needed) to write positions length .. length+n-1."""
        need = -(-(length + n) // self.page_size)
        new = max(0, need - len(table))
        cow = False
        if n > 0 and length % self.page_size and length // self.page_size < len(table):
            last = table[length // self.page_size]
            cow = last >= 0 and self.refs[last] > 1
        return new, cow


@dataclass
class _Request:
    length: int = 0                      # tokens whose keys/values (or state) are written
    tokens: List[int] = field(default_factory=list)
    slot: int = -1


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], max_requests: int = 64, share_prefixes: bool = False,
                 has_state: bool = False):
        # Prefix sharing is only sound when what a page holds is a pure function of the token
        # prefix for every mixer: no windows (pages vanish) and no per-request state.
        sound = share_prefixes and not has_state and all(g.window is None for g in groups)
        self.share_prefixes = sound
        self.groups = [_Group(g, sound) for g in groups]
        self.requests: Dict[object, _Request] = {}
        self.max_requests = max_requests
        self.free_slots: List[int] = list(range(max_requests - 1, -1, -1))
        self.fresh_slots: List[int] = []  # handed out since the last drain: to be zeroed on the device

    # ---------------------------------------------------------------------------------- queries
    def has(self, rid) -> bool:
        return rid in self.requests

    def length(self, rid) -> int:
        return self.requests[rid].length

    def slot_of(self, rid) -> int:
        return self.requests[rid].slot

    def table(self, group: int, rid) -> List[int]:
        return self.groups[group].tables[rid]

    def free_pages(self, group: int = 0) -> int:
        return self.groups[group].free_pages()

    def used_pages(self, group: int = 0) -> int:
        g = self.groups[group]
        return g.spec.num_pages - g.free_pages()

    def num_pages(self, group: int = 0) -> int:
        return self.groups[group].spec.num_pages

    def ref_count(self, group: int, page: int) -> int:
        return self.groups[group].refs[page]

    def slot(self, group: int, rid, pos: int) -> int:
        """Row of (request, position) in a cache layer of the group (kv.rs:199-201)."""
        g = self.groups[group]
        page = g.tables[rid][pos // g.page_size]
        assert page >= 0, "position lies on a page that was given back"
        return page * g.page_size + pos % g.page_size

    def drain_fresh_slots(self) -> List[int]:
        out, self.fresh_slots = self.fresh_slots, []
        return out

    def pages_needed(self, n_tokens: int, group: int = 0) -> int:
        return -(-n_tokens // self.groups[group].page_size)

    # ------------------------------------------------------------------------------ life cycle
    def add_request(self, rid, prompt: Sequence[int] = ()) -> int:
        """Start a request. With prefix sharing, whole leading pages whose token prefix is already
        cached are shared; never the page that holds the last prompt token, which must still run
        to give logits (kv.rs:135-157). Returns the number of tokens already present."""
        if rid in self.requests:
            raise ValueError(f"request {rid!r} exists")
        if not self.free_slots:
            raise OutOfPages("no free state slot")
        req = _Request(tokens=list(int(t) for t in prompt))
        req.slot = self.free_slots.pop()
        self.fresh_slots.append(req.slot)
        reused_pages = 0
        if self.share_prefixes and self.groups:
            ps = self.groups[0].page_size
            if all(g.page_size == ps for g in self.groups):
                found: List[List[int]] = []
                h = 0
                for i in range(len(req.tokens) // ps):
                    if (i + 1) * ps >= len(req.tokens):
                        break
                    h = chain_hash(h, req.tokens[i * ps:(i + 1) * ps])
                    pages = [g.by_hash.get(h) for g in self.groups]
                    if any(p is None for p in pages):
                        break
                    found.append(pages)
                reused_pages = len(found)
                for g in self.groups:
                    g.tables[rid] = []
                for pages in found:
                    for g, p in zip(self.groups, pages):
                        g.retain(p)
                        g.tables[rid].append(p)
                req.length = reused_pages * ps
        for g in self.groups:
            g.tables.setdefault(rid, [])
        self.requests[rid] = req
        return req.length

    def reserve(self, rid, n: int) -> List[Tuple[int, int, int]]:
        """Make room to write positions length .. length+n-1 in every group, all or nothing.
        Returns copy-on-write work as (group, source page, destination page) triples that the
        caller must carry out on the device before the step (kv.rs:161-196)."""
        req = self.requests[rid]
        plans = []
        for g in self.groups:
            new, cow = g.plan(g.tables[rid], req.length, n)
            if new + (1 if cow else 0) > g.free_pages():
                raise OutOfPages()
            plans.append((new, cow))
        copies = []
        for gi, (g, (new, cow)) in enumerate(zip(self.groups, plans)):
            table = g.tables[rid]
            if cow:
                i = req.length // g.page_size
                old = table[i]
                fresh = g.alloc()
                copies.append((gi, old, fresh))
                g.release(old)
                table[i] = fresh
            for _ in range(new):
                table.append(g.alloc())
        return copies

    def commit(self, rid, tokens: Sequence[int]) -> None:
        """Mark ``len(tokens)`` more positions as written; hash pages that became full
        (kv.rs:205-233); give back pages that a window has passed."""
        req = self.requests[rid]
        start = req.length
        req.length += len(tokens)
        if len(req.tokens) < req.length:
            del req.tokens[start:]
            req.tokens.extend(int(t) for t in tokens)
        for g in self.groups:
            table = g.tables[rid]
            if g.share:
                for bi in range(start // g.page_size, req.length // g.page_size):
                    p = table[bi]
                    if g.page_hash[p] is not None:
                        continue
                    h = 0
                    for c in range(bi + 1):
                        h = chain_hash(h, req.tokens[c * g.page_size:(c + 1) * g.page_size])
                    if h not in g.by_hash:
                        g.by_hash[h] = p
                        g.page_hash[p] = h
            if g.window is not None:
                for bi in range(min(g.first_live_page(req.length), len(table))):
                    if table[bi] >= 0:
                        g.release(table[bi])
                        table[bi] = -1

    def truncate(self, rid, length: int) -> None:
        """Forget everything after the first ``length`` tokens (kv.rs:237-257). Not available
        once a window has given pages back behind ``length``."""
        req = self.requests[rid]
        if length > req.length:
            raise ValueError("cannot truncate to more than is written")
        for g in self.groups:
            if g.window is not None and any(p < 0 for p in g.tables[rid][g.first_live_page(length):]):
                raise ValueError("a windowed group has already released pages that the shorter request would need")
        req.length = length
        del req.tokens[length:]
        for g in self.groups:
            table = g.tables[rid]
            keep = -(-length // g.page_size)
            dropped = table[keep:]
            del table[keep:]
            if length % g.page_size:
                p = table[length // g.page_size]
                if p >= 0 and g.refs[p] == 1 and g.page_hash[p] is not None:
                    g.by_hash.pop(g.page_hash[p], None)
                    g.page_hash[p] = None
            for p in dropped:
                if p >= 0:
                    g.release(p)

    def fork(self, parent, child) -> Tuple[int, int]:
        """New request sharing every page of ``parent`` (kv.rs:260-266). Its state slot is a
        copy, not a share: returns (parent slot, child slot) for the device copy."""
        if child in self.requests:
            raise ValueError(f"request {child!r} exists")
        if not self.free_slots:
            raise OutOfPages("no free state slot")
        src = self.requests[parent]
        req = _Request(length=src.length, tokens=list(src.tokens), slot=self.free_slots.pop())
        for g in self.groups:
            table = list(g.tables[parent])
            for p in table:
                if p >= 0:
                    g.retain(p)
            g.tables[child] = table
        self.requests[child] = req
        return src.slot, req.slot

    def free_request(self, rid) -> None:
        """Give back everything the request holds (kv.rs:268-274). Unknown ids are ignored."""
        req = self.requests.pop(rid, None)
        if req is None:
            return
        for g in self.groups:
            for p in g.tables.pop(rid):
                if p >= 0:
                    g.release(p)
        self.free_slots.append(req.slot)
        if req.slot in self.fresh_slots:
            self.fresh_slots.remove(req.slot)

    # ------------------------------------------------------------------------------ invariants
    def check_invariants(self) -> None:
        """Every page is referenced exactly as often as block tables name it; pages nobody names
        are exactly the free and the cached ones, each once; slots likewise (kv.rs:278-288)."""
        for gi, g in enumerate(self.groups):
            want = [0] * g.spec.num_pages
            for table in g.tables.values():
                for p in table:
                    if p >= 0:
                        want[p] += 1
            assert want == g.refs, f"group {gi}: page reference counts drifted"
            idle = [p for p, r in enumerate(g.refs) if r == 0]
            pool = g.free + g.cached
            assert len(pool) == len(set(pool)), f"group {gi}: a page is on the free lists twice"
            assert sorted(pool) == idle, f"group {gi}: free lists drifted from the reference counts"
            assert all(g.page_hash[p] is not None for p in g.cached), f"group {gi}: cached page without a hash"
            assert all(g.page_hash[p] is None for p in g.free), f"group {gi}: free page still hashed"
            for h, p in g.by_hash.items():
                assert g.page_hash[p] == h, f"group {gi}: hash index drifted"
            assert set(g.tables) == set(self.requests), f"group {gi}: tables and requests differ"
        held = sorted(r.slot for r in self.requests.values())
        assert len(held) == len(set(held)), "a state slot is held twice"
        assert sorted(held + self.free_slots) == list(range(self.max_requests)), "state slots drifted"
