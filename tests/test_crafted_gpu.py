"""Crafted models in which every logit says which keys a row read: a far key among hundreds, the
edges of a window, the edges of pages, pages that are used again. Random weights would average
such faults away below any bfloat16 tolerance; here a misread key moves a logit by about 0.1 or
more while rounding stays below 0.02, in float32 and in bfloat16 alike."""
import random

import numpy as np
import pytest
import torch

import replay_util as ru
import toy_arch

pytestmark = pytest.mark.gpu

ATOL = {"float32": 1e-4, "bfloat16": 2e-2}


def engine_for(folder, dtype, tokens, page_size=16):
    from glassbox_b200.engine.engine import Engine
    return Engine(folder, dtype, cache_tokens=tokens, page_size=page_size, max_batch_tokens=512, max_requests=8)


def check(info, got, requests, dtype, what):
    n = info["nh"] * info["hd"]
    for rid, toks in requests.items():
        truth = toy_arch.probe_truth(info, toks)
        have = got.get(rid, {})
        assert have, f"{what}: nothing came back for {rid}"
        for p in sorted(have):
            diff = np.abs(have[p][:n] - truth[p])
            assert diff.max() <= ATOL[dtype], \
                f"{what}: {rid} position {p} head {int(diff.argmax()) // info['hd']}: off by {diff.max():.3f} ({dtype})"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [None, 37])
def test_every_row_reads_exactly_its_keys(tmp_path, dtype, window):
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    info = toy_arch.write_probe_model(str(tmp_path / "m"), window=window, store=store, seed=1)
    rng = random.Random(2)
    requests = {f"r{i}": [rng.randrange(info["vocab"]) for _ in range(n)] for i, n in enumerate([300, 65, 130, 17, 240, 48])}
    eng = engine_for(str(tmp_path / "m"), dtype, 1024)
    for label, steps in (("whole", ru.whole(requests)), ("tail", ru.tail_one_by_one(requests)),
                         ("portions", ru.changing_portions(requests))):
        check(info, ru.run_steps_inprocess(eng, steps), requests, dtype, f"window {window} {label}")
    for seed in (1, 2, 3):
        steps = ru.mixed(requests, random.Random(seed))
        need = ru.live_tokens_needed(steps)
        small = engine_for(str(tmp_path / "m"), dtype, need)       # so few pages that they are used again
        check(info, ru.run_steps_inprocess(small, steps), requests, dtype, f"window {window} mixed {seed}")
        assert small.cache.free_pages() == small.cache.num_pages()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_far_key_among_hundreds(tmp_path, dtype):
    """Position 3 holds the only key that the last rows' queries match; everything between is filler."""
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    info = toy_arch.write_probe_model(str(tmp_path / "m"), store=store, seed=5, nh=3, nkv=1, hd=16, vocab=300)
    kd, qd = info["kdir"][:, 0], info["qdir"]
    needle_dir = 7
    needle = next(t for t in range(300) if kd[t] == needle_dir)
    seekers = [t for t in range(300) if all(qd[t, h] == needle_dir for h in range(1)) and kd[t] != needle_dir]
    fillers = [t for t in range(300) if kd[t] != needle_dir and (qd[t] != needle_dir).all()]
    rng = random.Random(0)
    toks = [rng.choice(fillers) for _ in range(400)]
    toks[3] = needle
    for p in (250, 399):
        toks[p] = seekers[0]
    truth = toy_arch.probe_truth(info, toks)
    # head 0 of the seekers must return the needle's value vector, exactly that key alone
    assert np.allclose(truth[399][:16] - info["had"][needle_dir], info["val"][needle, 0])
    eng = engine_for(str(tmp_path / "m"), dtype, 448)
    requests = {"a": toks}
    for label, steps in (("whole", ru.whole(requests)), ("tail", ru.tail_one_by_one(requests)),
                         ("portions", ru.changing_portions(requests))):
        check(info, ru.run_steps_inprocess(eng, steps), requests, dtype, label)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [16, 32])
def test_window_edge_and_page_edges(tmp_path, dtype, page_size):
    """Matching keys sit just inside and just outside the window of the query, and on both sides of
    page boundaries; the query's row must count exactly the inside ones."""
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    w = 37
    info = toy_arch.write_probe_model(str(tmp_path / "m"), store=store, seed=9, window=w, nh=2, nkv=2, hd=16, vocab=300)
    kd, qd = info["kdir"], info["qdir"]
    d0 = 5
    key_tokens = [t for t in range(300) if kd[t, 0] == d0 and kd[t, 1] == d0][:1] or \
                 [t for t in range(300) if kd[t, 0] == d0][:1]
    ask = next(t for t in range(300) if qd[t, 0] == d0 and kd[t, 0] != d0)
    fillers = [t for t in range(300) if kd[t, 0] != d0 and qd[t, 0] != d0]
    rng = random.Random(1)
    for t_query in (100, 111, 112, 113, 127, 128):
        toks = [rng.choice(fillers) for _ in range(t_query + 1)]
        toks[t_query] = ask
        for p in (t_query - w, t_query - w + 1, t_query - w + 2, 15, 16, 17, t_query - 1):
            toks[p] = key_tokens[0]
        requests = {"a": toks}
        eng = engine_for(str(tmp_path / "m"), dtype, 192, page_size=page_size)
        for label, steps in (("whole", ru.whole(requests)), ("tail", ru.tail_one_by_one(requests, tail=20)),
                             ("portions", ru.changing_portions(requests))):
            check(info, ru.run_steps_inprocess(eng, steps), requests, dtype, f"query at {t_query} {label}")


@pytest.mark.parametrize("window", [None, 37])
def test_mixed_batches_split_between_the_decode_and_the_flash_kernel(tmp_path, monkeypatch, window):
    """A batch that starts with single-token requests and goes on with prompt portions is served by two
    attention kernels (here forced for any such batch; in service only for large ones): every row must still
    read exactly its keys."""
    from glassbox_b200.parts import attention
    monkeypatch.setattr(attention, "SPLIT_MIXED_ABOVE", 0)
    split_calls = []
    real = attention.GqaAttention._attend_decode

    def counting(self, ctx, q, att, cache, n):
        if not ctx.decode_only:
            split_calls.append((n, ctx.n))
        return real(self, ctx, q, att, cache, n)
    monkeypatch.setattr(attention.GqaAttention, "_attend_decode", counting)
    info = toy_arch.write_probe_model(str(tmp_path / "m"), window=window, store=torch.bfloat16, seed=3, hd=64, nh=2, nkv=1)
    rng = random.Random(4)
    requests = {f"r{i}": [rng.randrange(info["vocab"]) for _ in range(n)] for i, n in enumerate([300, 65, 150, 40, 200, 90])}
    for seed in (1, 2):
        steps = ru.mixed(requests, random.Random(seed))
        for st in steps:                                   # the scheduler's order: single tokens first
            st["entries"].sort(key=lambda e: len(e["tokens"]) > 1)
        eng = engine_for(str(tmp_path / "m"), "bfloat16", ru.live_tokens_needed(steps))
        check(info, ru.run_steps_inprocess(eng, steps), requests, "bfloat16", f"window {window} split mixed {seed}")
    assert any(0 < k < n for k, n in split_calls), "no batch was split: the test did not reach what it is about"


@pytest.mark.parametrize("share", [False, True], ids=["no-sharing", "share-prefixes"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_forks_preemption_and_shared_prefixes_read_exactly_their_keys(tmp_path, monkeypatch, dtype, share):
    """The same trace of cache operations as the replay test, on the probe model, where a key read from the wrong
    page (a copy that did not run, a page taken over from another request) shows at full size in bfloat16 too."""
    from glassbox_b200.engine.engine import Engine
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    info = toy_arch.write_probe_model(str(tmp_path / "m"), store=store, seed=4)
    for seed in (1, 2):
        steps, known = ru.forks_preemption_and_shared_prefix(info["vocab"], random.Random(seed))
        eng = Engine(str(tmp_path / "m"), dtype, cache_tokens=ru.live_tokens_needed(steps), max_batch_tokens=512,
                     max_requests=8, share_prefixes=share)
        got = ru.run_steps_inprocess(eng, steps)
        check(info, got, known, dtype, f"forks/preemption seed {seed}")
        assert sum(len(v) for v in got.values()) == sum(len(e["want"]) for s in steps for e in s["entries"])
        if share:
            assert eng.cache.share_prefixes
    # the test must be able to fail: without the copy that a write into a shared page needs, the fork's rows
    # (or its parent's) read keys that the other wrote
    steps, known = ru.forks_preemption_and_shared_prefix(info["vocab"], random.Random(1))
    eng = Engine(str(tmp_path / "m"), dtype, cache_tokens=ru.live_tokens_needed(steps), max_batch_tokens=512, max_requests=8)
    monkeypatch.setattr(eng, "run_copies", lambda copies: None)
    got = ru.run_steps_inprocess(eng, steps)
    with pytest.raises(AssertionError):
        check(info, got, known, dtype, "without copies")
