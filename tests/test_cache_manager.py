"""The cache manager on the CPU: no page lost, held twice or freed twice; prefix sharing,
copy-on-write, fork, truncate, windows, state slots; random orders of requests.
Unit cases mirror crates/glassbox-core/src/kv.rs:295-349."""
import random

import pytest

from glassbox_b200.cache import CacheManager, GroupSpec, OutOfPages, chain_hash


def mgr(pages=8, share=True, window=None, max_requests=8, page_size=16, groups=1):
    return CacheManager([GroupSpec(pages, page_size, window) for _ in range(groups)], max_requests=max_requests,
                        share_prefixes=share)


def feed(m, rid, tokens):
    m.reserve(rid, len(tokens))
    m.commit(rid, tokens)


def test_chain_hash_is_fnv1a_over_le_bytes():
    h = 0 ^ 0xCBF29CE484222325
    for b in (7).to_bytes(4, "little"):
        h = ((h ^ b) * 0x100000001B3) & (2 ** 64 - 1)
    assert chain_hash(0, [7]) == h
    assert chain_hash(chain_hash(0, [1, 2]), [3]) != chain_hash(0, [1, 2, 3])


def plain_fnv(prev, tokens):
    h = (prev ^ 0xCBF29CE484222325) & (2 ** 64 - 1)
    for t in tokens:
        for b in int(t).to_bytes(4, "little"):
            h = ((h ^ b) * 0x100000001B3) & (2 ** 64 - 1)
    return h


def test_full_pages_are_indexed_under_the_chain_of_their_prefix():
    m = mgr(pages=6, share=True)
    toks = list(range(100, 100 + 40))
    m.add_request("a", toks)
    feed(m, "a", toks[:35])                      # two full pages and a partial one, in one commit
    t = m.table(0, "a")
    h0 = plain_fnv(0, toks[:16])
    assert m.page_hash(0, t[0]) == h0 and m.page_hash(0, t[1]) == plain_fnv(h0, toks[16:32])
    assert m.page_hash(0, t[2]) is None
    feed(m, "a", toks[35:40])                    # the third page is still not full
    assert m.page_hash(0, t[2]) is None
    m.check_invariants()


def test_pages_come_in_order_and_go_back():
    m = mgr(pages=4, share=False)
    m.add_request("a")
    feed(m, "a", list(range(20)))
    assert m.table(0, "a") == [0, 1] and m.slot(0, "a", 17) == 16 + 1
    assert m.free_pages() == 2
    m.free_request("a")
    assert m.free_pages() == 4
    m.check_invariants()


def test_prefix_pages_are_shared_and_freed():
    m = mgr(pages=8)
    prompt = list(range(40))
    assert m.add_request(1, prompt) == 0
    feed(m, 1, prompt)
    assert m.add_request(2, prompt) == 32          # two whole pages; the last token must still run
    assert m.table(0, 2) == m.table(0, 1)[:2]
    assert m.ref_count(0, m.table(0, 1)[0]) == 2
    # a prompt that is exactly two pages long may only reuse one: its last token has to run
    assert m.add_request(3, prompt[:32]) == 16
    m.check_invariants()
    for r in (1, 2, 3):
        m.free_request(r)
    assert m.free_pages() == 8                     # cached pages count as free
    m.check_invariants()
    assert m.add_request(4, prompt) == 32          # ... and are found again until evicted
    m.check_invariants()


def test_cached_pages_are_evicted_oldest_first_when_space_is_needed():
    m = mgr(pages=3)
    m.add_request(1, list(range(33)))
    feed(m, 1, list(range(33)))
    m.free_request(1)                              # pages 0,1 cached (hashed), page 2 free
    m.add_request(2)
    feed(m, 2, [9] * 48)                           # needs all three pages: evicts both cached ones
    m.check_invariants()
    m.free_request(2)
    assert m.add_request(3, list(range(33))) == 0  # the old prefix is gone
    m.check_invariants()


def test_fork_copies_on_write():
    m = mgr(pages=6, share=False)
    m.add_request("p")
    feed(m, "p", list(range(20)))
    m.fork("p", "c")
    assert m.table(0, "c") == m.table(0, "p")
    copies = m.reserve("c", 1)                     # the shared partial page must become private
    assert len(copies) == 1 and copies[0][1] == m.table(0, "p")[1] and copies[0][2] == m.table(0, "c")[1]
    assert m.table(0, "c")[0] == m.table(0, "p")[0] and m.table(0, "c")[1] != m.table(0, "p")[1]
    assert m.slot_of("c") != m.slot_of("p")
    m.commit("c", [99])
    assert m.reserve("p", 1) == []                 # the parent is alone on its page again
    m.check_invariants()
    m.free_request("p")
    m.free_request("c")
    assert m.free_pages() == 6


def test_reserve_is_all_or_nothing_and_counts_the_cow_page():
    m = mgr(pages=3, share=False)
    m.add_request("p")
    feed(m, "p", list(range(20)))                  # two pages
    m.fork("p", "c")
    before = (list(m.table(0, "c")), m.free_pages())
    with pytest.raises(OutOfPages):
        m.reserve("c", 16)                         # one copy + one new page, only one page free
    assert (m.table(0, "c"), m.free_pages()) == before
    m.check_invariants()


def test_truncate_unregisters_a_rewritten_hashed_page():
    m = mgr(pages=4)
    m.add_request(1)
    feed(m, 1, list(range(32)))
    m.truncate(1, 20)                              # page 1 is partial again and will be overwritten
    feed(m, 1, [7] * 12)
    m.free_request(1)
    assert m.add_request(2, list(range(40))) == 16  # page 0's prefix survives, page 1's stale hash does not
    m.check_invariants()


def test_window_gives_pages_back_early():
    m = mgr(pages=4, window=20, share=False)
    m.add_request("a")
    for _ in range(100):                           # far more tokens than 4 pages hold
        feed(m, "a", [1])
        m.check_invariants()
    table = m.table(0, "a")
    assert len(table) == 7 and table[:5] == [-1] * 5 and all(p >= 0 for p in table[5:])
    # a query at position >= 100 sees keys 81..: page 5 (tokens 80..95) must still be there
    assert m.used_pages() == 2
    m.free_request("a")
    assert m.free_pages() == 4


def test_window_keeps_what_a_long_portion_needs():
    m = mgr(pages=8, window=8, share=False)
    m.add_request("a")
    m.reserve("a", 100)                            # every row of the portion needs its own window
    assert all(p >= 0 for p in m.table(0, "a")) and len(m.table(0, "a")) == 7
    m.commit("a", [0] * 100)
    assert m.table(0, "a")[:5] == [-1] * 5
    m.check_invariants()


def test_groups_have_pages_of_their_own():
    m = CacheManager([GroupSpec(8, 16, None), GroupSpec(3, 16, 16)], max_requests=4)
    m.add_request("a")
    for _ in range(60):
        feed(m, "a", [1])
    assert m.used_pages(0) == 4 and m.used_pages(1) <= 2
    m.add_request("b")
    with pytest.raises(OutOfPages):
        m.reserve("b", 48)                         # fits group 0, not the small windowed group
    assert m.table(0, "b") == [] and m.table(1, "b") == []
    m.check_invariants()


def test_prefix_sharing_is_off_when_unsound():
    assert not CacheManager([GroupSpec(8, 16, 32)], share_prefixes=True).share_prefixes
    assert not CacheManager([GroupSpec(8, 16, None)], share_prefixes=True, has_state=True).share_prefixes


def test_state_slots():
    m = mgr(pages=8, max_requests=2, share=False)
    m.add_request("a")
    m.add_request("b")
    assert sorted(m.drain_fresh_slots()) == [0, 1] and m.drain_fresh_slots() == []
    with pytest.raises(OutOfPages):
        m.add_request("c")
    m.free_request("a")
    m.add_request("c")
    assert m.drain_fresh_slots() == [m.slot_of("c")]
    m.check_invariants()


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window, share", [(None, True), (None, False), (24, False)])
def test_random_orders_never_lose_or_double_a_page(seed, window, share):
    rng = random.Random(seed)
    m = mgr(pages=12, share=share, window=window, max_requests=6)
    live, next_id = {}, 0
    shared = [rng.randrange(50) for _ in range(40)]
    for _ in range(400):
        op = rng.random()
        try:
            if op < 0.2 and len(live) < 6:
                prompt = (shared[:rng.choice([16, 32, 40])] if rng.random() < 0.5 else []) + \
                    [rng.randrange(50) for _ in range(rng.randrange(1, 30))]
                reused = m.add_request(next_id, prompt)
                assert reused % 16 == 0 and reused < len(prompt)
                live[next_id] = prompt[reused:]
                next_id += 1
            elif op < 0.7 and live:
                rid = rng.choice(list(live))
                pending = live[rid]
                n = rng.randrange(1, 20)
                chunk = pending[:n] if pending else [rng.randrange(50) for _ in range(1)]
                m.reserve(rid, len(chunk))
                m.commit(rid, chunk)
                live[rid] = pending[len(chunk):]
            elif op < 0.8 and live and len(live) < 6:
                parent = rng.choice(list(live))
                m.fork(parent, next_id)
                live[next_id] = list(live[parent])
                next_id += 1
            elif op < 0.85 and live and window is None:
                rid = rng.choice(list(live))
                m.truncate(rid, rng.randrange(0, m.length(rid) + 1))
                live[rid] = []
            elif live:
                rid = rng.choice(list(live))
                m.free_request(rid)
                del live[rid]
        except OutOfPages:
            pass
        m.check_invariants()
    for rid in list(live):
        m.free_request(rid)
    m.check_invariants()
    assert m.free_pages() == 12 and len(m.free_slots) == 6


def test_the_metadata_block_of_a_padded_step():
    """Two single-token requests, padding up to four, a three-token portion, one trailing padding sequence:
    positions, row -> sequence, first rows, start positions (-1 for padding), slots, tables and wanted rows."""
    import numpy as np
    m = mgr(pages=8, share=False)
    for rid, have in (("a", 17), ("b", 3), ("c", 30)):
        m.add_request(rid)
        feed(m, rid, list(range(have)))
    for rid, n in (("a", 1), ("b", 1), ("c", 3)):
        m.reserve(rid, n)
    n, S, n_want, P = 12, 6, 8, 4
    sizes = [n, n, n, n_want, S + 1, S, S, n_want, n, n, S * P]
    off = np.concatenate(([0], np.cumsum(sizes)[:-1])).astype(np.int64)
    host = np.full(int(sum(sizes)), 77, dtype=np.int32)
    info, longest = m.fill_step(["a", "b", "c"], np.array([1, 1, 3], dtype=np.int32), np.array([5, 6, 7, 8, 9], dtype=np.int32),
                                np.array([1, 1, 1], dtype=np.int32), np.array([0, 0, 2], dtype=np.int32), n, S, n_want, P, off,
                                host, np.array([1, 0, 1], dtype=np.uint8), lead=2, pad_after=2,
                                feedback_mask=np.array([0, 1, 1], dtype=np.uint8))
    sec = lambda i: host[off[i]:off[i] + sizes[i]]
    assert longest == 33 and info.tolist() == [[17, m.slot_of("a"), 0], [3, m.slot_of("b"), 1], [30, m.slot_of("c"), 4]]
    assert sec(0)[:7].tolist() == [5, 6, 0, 0, 7, 8, 9]                                   # tokens; padding rows hold 0
    assert sec(1).tolist() == [17, 3, -1, -1, 30, 31, 32, -1, -1, -1, -1, -1]             # positions
    assert sec(2).tolist() == [0, 1, 2, 3, 4, 4, 4, 5, 5, 5, 5, 5]                         # row -> sequence
    assert sec(4).tolist() == [0, 1, 2, 3, 4, 7, 8]                                        # first rows, and the end
    assert sec(5).tolist() == [17, 3, -1, -1, 30, -1]                                      # start positions
    assert sec(3).tolist() == [0, 1, 6, 2, 3, 7, 0, 0]       # wanted: a, b, c's third row, then padding rows, then row 0
    ta, tc = m.table(0, "a"), m.table(0, "c")
    assert sec(7).tolist() == [m.slot_of("a"), -1, m.slot_of("c"), -1, -1, -1, -1, -1]     # who is sampled from its own state
    # whose token comes from the device: b's one row; c brings three tokens, so its flag does not apply
    assert sec(8).tolist() == [-1, m.slot_of("b"), -1, -1, -1, -1, -1, -1, -1, -1, -1, -1]
    assert sec(9).tolist() == [ta[1] * 16 + 1, m.table(0, "b")[0] * 16 + 3, -1, -1, tc[1] * 16 + 14, tc[1] * 16 + 15,
                               tc[2] * 16 + 0, -1, -1, -1, -1, -1]                         # cache slot of every row
    tables = sec(10).reshape(S, P)
    assert tables[0, :2].tolist() == ta and tables[4, :3].tolist() == tc and (tables[2:4] == -1).all() and (tables[5] == -1).all()


def test_a_write_into_a_hashed_page_held_alone_drops_its_hash():
    """Fork, the child truncates into a hashed page (still shared, so its hash stays), the parent goes away, the
    child writes without a copy: the page's old hash must not outlive its contents."""
    m = mgr(pages=6)
    prompt = list(range(40))
    m.add_request("p", prompt)
    feed(m, "p", prompt)                           # pages 0 and 1 full and hashed
    m.fork("p", "c")
    m.truncate("c", 20)                            # into page 1, which the parent still holds
    page1 = m.table(0, "c")[1]
    assert m.page_hash(0, page1) is not None       # still valid for the parent
    m.free_request("p")
    assert m.reserve("c", 5) == []                 # alone on the page: no copy
    assert m.page_hash(0, page1) is None           # and the index has forgotten it
    m.commit("c", [7] * 5)
    m.check_invariants()
    m.free_request("c")
    assert m.add_request("again", prompt) == 16    # only the untouched first page is found again
    m.check_invariants()


def test_commit_records_the_tokens_that_ran_not_the_ones_expected():
    m = mgr(pages=6)
    m.add_request("a", list(range(100, 140)))      # expected
    feed(m, "a", [5] * 33)                         # what really ran
    assert m.tokens("a") == [5] * 33
    m.free_request("a")
    assert m.add_request("b", list(range(100, 140))) == 0, "a page was indexed under tokens it never held"
    m.free_request("b")
    assert m.add_request("c", [5] * 40) == 32
    m.check_invariants()


def test_a_preempted_request_takes_its_copy_on_write_work_with_it():
    """Three requests; the last admitted is a fork that decodes, so it is planned first and its write into the
    shared partial page needs a copy. The prompt portion planned after it runs out of pages, the fork is preempted,
    and its copy must go with it: the destination page is back in the pool and is handed out again in the same plan."""
    m = mgr(pages=5, share=False)
    m.add_request("p")
    feed(m, "p", list(range(20)))                  # 2 pages
    m.add_request("q")
    feed(m, "q", list(range(16)))                  # 1 page, full
    m.fork("p", "c")                               # shares p's 2 pages; 2 pages free
    # c decodes (planned first, copies page 1 into a fresh page), p brings 5 tokens (fits its page), q's
    # portion of 32 tokens needs 2 pages where 1 is left: c, admitted last, is preempted
    plan, copies, preempted, lone = m.plan_step(["p", "q", "c"], [5, 32, 1], 64)
    assert preempted == 1 and not lone and plan == [(0, 5), (1, 32)]
    assert copies == [], "a copy for the preempted request was kept"
    assert m.length("c") == -1
    m.free_request("c")
    assert len(set(m.table(0, "p")) | set(m.table(0, "q"))) == 5 and m.free_pages() == 0
    m.check_invariants()
