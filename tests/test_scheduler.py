"""The scheduler's decisions, on the CPU with a stand-in backend. Property tests mirror
crates/glassbox-server/tests/scheduler.rs:84-186: batching, chunked prefill, preemption, aborts and
prefix sharing never change what a request generates and never leak a page."""
import random

import pytest

from glassbox_b200.engine.scheduler import ABORTED, LENGTH, STOP, Request, Scheduler, SchedulerConfig
from glassbox_b200.sampling import SamplerConfig

from plain.backend import PlainBackend
from plain.llama_plain import greedy


def run_all(backend, config, jobs, trace=False):
    s = Scheduler(backend, config, trace=trace)
    ids = [s.submit(Request(prompt=p, max_tokens=n)) for p, n in jobs]
    guard = 0
    while not s.is_idle():
        s.step()
        backend.cache.check_invariants()
        guard += 1
        assert guard < 10_000, "the scheduler made no progress"
    assert backend.cache.free_pages() == backend.cache.num_pages(), "pages leaked"
    assert len(backend.cache.free_slots) == backend.cache.max_requests, "state slots leaked"
    return [s.finished[i] for i in ids], s


def random_jobs(seed, count, vocab, max_len=60, tokens=None):
    rng = random.Random(seed)
    return [([rng.randrange(vocab) for _ in range(rng.randrange(1, max_len))], tokens or rng.randrange(1, 12))
            for _ in range(count)]


def test_decodes_go_first_and_prompts_are_cut_under_the_budget(model_dirs):
    folder = model_dirs("A")
    backend = PlainBackend(folder, num_pages=64)
    s = Scheduler(backend, SchedulerConfig(token_budget=16, max_seqs=4))
    a = s.submit(Request(prompt=list(range(1, 6)), max_tokens=4))       # 5 tokens: whole in step 1
    b = s.submit(Request(prompt=list(range(1, 41)), max_tokens=2))      # 40 tokens: cut into portions
    s.step()
    assert backend.step_log[-1] == [(a, 5, [4]), (b, 11, [])]            # budget 16 = 5 + 11
    s.step()
    assert backend.step_log[-1] == [(a, 1, [0]), (b, 15, [])]            # the decoding request first, one token
    s.step()
    assert backend.step_log[-1] == [(a, 1, [0]), (b, 14, [13])]          # prompt ends: logits wanted at its last row
    s.run_until_idle()
    assert s.finished[a].reason == LENGTH and len(s.finished[a].tokens) == 4
    assert len(s.finished[b].tokens) == 2


def test_max_seqs_and_fifo_admission(model_dirs):
    backend = PlainBackend(model_dirs("A"), num_pages=64)
    s = Scheduler(backend, SchedulerConfig(token_budget=64, max_seqs=2))
    ids = [s.submit(Request(prompt=[1, 2, 3], max_tokens=2)) for _ in range(4)]
    s.step()
    assert [e[0] for e in backend.step_log[-1]] == ids[:2] and len(s.waiting) == 2
    s.run_until_idle()
    assert all(len(s.finished[i].tokens) == 2 for i in ids)


@pytest.mark.parametrize("seed", range(3))
def test_batched_equals_unbatched(model_dirs, seed):
    folder = model_dirs("A")
    jobs = random_jobs(seed, 6, 256, max_len=40)
    outs, _ = run_all(PlainBackend(folder, num_pages=256), SchedulerConfig(token_budget=16, max_seqs=4), jobs)
    for (p, n), out in zip(jobs, outs):
        assert out.tokens == greedy(folder, p, n)


def test_preemption_keeps_outputs_and_frees_pages(model_dirs):
    folder = model_dirs("A")
    jobs = random_jobs(99, 8, 256, max_len=40, tokens=20)
    # 9 pages = 144 token slots for 8 requests that each need 2-4: pages run out
    outs, s = run_all(PlainBackend(folder, num_pages=9), SchedulerConfig(token_budget=64, max_seqs=8), jobs, trace=True)
    assert s.metrics.preemptions > 0, "the test did not exercise preemption"
    for (p, n), out in zip(jobs, outs):
        assert out.tokens == greedy(folder, p, n)
    # the victim is always the most recently admitted request, and it returns to the front
    assert any(r["preempted"] for r in s.trace)


def test_preempted_request_goes_to_the_front_and_waits_for_its_whole_context(model_dirs):
    backend = PlainBackend(model_dirs("A"), num_pages=4, share_prefixes=False)
    s = Scheduler(backend, SchedulerConfig(token_budget=64, max_seqs=2), trace=True)
    a = s.submit(Request(prompt=[1] * 30, max_tokens=10))     # 2 pages, grows into a third
    b = s.submit(Request(prompt=[2] * 14, max_tokens=30))     # 1 page, grows into a second
    c = s.submit(Request(prompt=[3] * 5, max_tokens=3))       # queued behind
    s.step()
    assert [x.id for x in s.running] == [a, b] and [x.id for x in s.waiting] == [c]
    while s.metrics.preemptions == 0:
        s.step()
    assert s.trace[-1]["preempted"] == [b], "the most recently admitted request is the victim"
    assert [x.id for x in s.waiting] == [b, c], "the preempted request waits in front of later arrivals"
    s.step()
    assert [x.id for x in s.running] == [a], "it stays out until its whole context plus a page fits"
    s.run_until_idle()
    assert {s.finished[i].reason for i in (a, b, c)} == {LENGTH}
    assert len(s.finished[b].tokens) == 30 and len(s.finished[c].tokens) == 3


def test_a_lone_request_that_cannot_fit_ends_with_length(model_dirs):
    backend = PlainBackend(model_dirs("A"), num_pages=2)
    outs, s = run_all(backend, SchedulerConfig(token_budget=64, max_seqs=4), [([5] * 20, 50)])
    # 32 slots hold the prompt and 12 generated tokens; the 13th is sampled from the last slot's
    # logits and cannot be fed any more
    assert outs[0].reason == LENGTH and len(outs[0].tokens) == 13
    outs, _ = run_all(PlainBackend(model_dirs("A"), num_pages=1), SchedulerConfig(), [([5] * 20, 5)])
    assert outs[0].reason == LENGTH and outs[0].tokens == []             # not even the prompt fits


def test_stop_tokens_max_tokens_zero_and_max_position(model_dirs):
    folder = model_dirs("A")
    backend = PlainBackend(folder, num_pages=64)
    s = Scheduler(backend, SchedulerConfig())
    free = greedy(folder, [7, 8, 9], 6)
    stop_at = free[3]
    a = s.submit(Request(prompt=[7, 8, 9], max_tokens=6, stop=[stop_at]))
    z = s.submit(Request(prompt=[1, 2], max_tokens=0))
    long = s.submit(Request(prompt=list(range(1, 120)), max_tokens=100))   # max_position is 128
    s.run_until_idle()
    assert s.finished[a].reason == STOP and s.finished[a].tokens == free[:free.index(stop_at)]
    assert s.finished[z].reason == LENGTH and s.finished[z].tokens == []
    assert s.finished[long].reason == LENGTH and len(s.finished[long].tokens) == 128 - 119
    assert backend.cache.free_pages() == 64


def test_aborts_free_everything(model_dirs):
    backend = PlainBackend(model_dirs("A"), num_pages=32)
    s = Scheduler(backend, SchedulerConfig(token_budget=16, max_seqs=4))
    rng = random.Random(4)
    ids = [s.submit(Request(prompt=p, max_tokens=n)) for p, n in random_jobs(4, 8, 256, max_len=30)]
    steps = 0
    while not s.is_idle():
        s.step()
        steps += 1
        if steps % 3 == 0:
            s.abort(rng.choice(ids))                 # running, waiting or already finished
        backend.cache.check_invariants()
    assert backend.cache.free_pages() == 32
    assert any(f.reason == ABORTED for f in s.finished.values())


def test_prefix_sharing_never_changes_outputs(model_dirs):
    folder = model_dirs("A")
    rng = random.Random(8)
    prefix = [rng.randrange(256) for _ in range(70)]
    jobs = [(prefix + [rng.randrange(256) for _ in range(rng.randrange(1, 10))], 4) for _ in range(4)]
    on, s_on = run_all(PlainBackend(folder, num_pages=64, share_prefixes=True),
                       SchedulerConfig(token_budget=32, max_seqs=2), jobs)
    off, s_off = run_all(PlainBackend(folder, num_pages=64, share_prefixes=False),
                         SchedulerConfig(token_budget=32, max_seqs=2), jobs)
    assert [o.tokens for o in on] == [o.tokens for o in off]
    assert s_on.metrics.prefix_hit_tokens >= 64 and s_off.metrics.prefix_hit_tokens == 0


def test_temperature_sampling_is_seeded_per_request(model_dirs):
    folder = model_dirs("B")
    def run():
        s = Scheduler(PlainBackend(folder, num_pages=64), SchedulerConfig(token_budget=16))
        ids = [s.submit(Request(prompt=[3, 1, 4, 1, 5], max_tokens=8, sampler=SamplerConfig(temperature=0.8, seed=k)))
               for k in (1, 2, 1)]
        s.run_until_idle()
        return [s.finished[i].tokens for i in ids]
    a, b = run(), run()
    assert a == b and a[0] == a[2] and a[0] != a[1]


def test_the_native_plan_of_a_step_decodes_first_fills_the_budget_and_preempts_the_latest():
    from glassbox_b200.cache import CacheManager, GroupSpec
    m = CacheManager([GroupSpec(8, 16)], max_requests=8, share_prefixes=False)
    for rid, have in (("a", 20), ("b", 0), ("c", 33)):          # a and c decode; b still has its prompt to run
        m.add_request(rid)
        if have:
            m.reserve(rid, have)
            m.commit(rid, list(range(have)))
    # 8 pages: a holds 2, c holds 3; b may take what fits the budget
    plan, copies, preempted, lone = m.plan_step(["a", "b", "c"], [1, 500, 1], 34)
    assert plan == [(0, 1), (2, 1), (1, 32)] and not copies and preempted == 0 and not lone
    m.commit("a", [1]); m.commit("c", [1]); m.commit("b", list(range(32)))
    m.check_invariants()
    assert m.free_pages() == 1
    # the next portion of b needs 2 pages, one is free: c, admitted last, gives way (its 3 pages come back)
    plan, copies, preempted, lone = m.plan_step(["a", "b", "c"], [1, 468, 1], 34)
    assert preempted == 1 and not lone and plan == [(0, 1), (1, 32)]
    assert m.length("c") == -1                                   # the library has forgotten it
    m.free_request("c")                                          # and now the wrapper has too
    m.check_invariants()
    # a lone request that cannot fit is reported, nothing is reserved for it
    lone_m = CacheManager([GroupSpec(2, 16)], max_requests=2, share_prefixes=False)
    lone_m.add_request("x")
    plan, copies, preempted, lone = lone_m.plan_step(["x"], [100], 64)
    assert lone and plan == [] and preempted == 0 and lone_m.free_pages() == 2


def test_an_over_long_prompt_is_refused_at_the_door_and_harms_nobody(model_dirs):
    folder = model_dirs("A")                                              # max_position 128
    backend = PlainBackend(folder, num_pages=64)
    s = Scheduler(backend, SchedulerConfig(token_budget=32, max_seqs=4))
    ok = [s.submit(Request(prompt=[3, 4, 5], max_tokens=3)), s.submit(Request(prompt=list(range(1, 60)), max_tokens=2))]
    with pytest.raises(ValueError, match="max_position"):
        s.submit(Request(prompt=[1] * 129, max_tokens=4))
    edge = s.submit(Request(prompt=[2] * 128, max_tokens=4))              # fills the context exactly: one token, then length
    s.run_until_idle()
    assert s.finished[ok[0]].tokens == greedy(folder, [3, 4, 5], 3)
    assert len(s.finished[ok[1]].tokens) == 2
    assert s.finished[edge].reason == LENGTH and len(s.finished[edge].tokens) == 1
    backend.cache.check_invariants()
    assert backend.cache.free_pages() == 64


def test_fork_shares_the_parents_pages_and_goes_its_own_way(model_dirs):
    folder = model_dirs("B")
    backend = PlainBackend(folder, num_pages=16, share_prefixes=False)
    s = Scheduler(backend, SchedulerConfig(token_budget=64, max_seqs=4))
    prompt = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5, 8, 9, 7, 9, 3, 2, 3, 8, 4, 6]
    parent = s.submit(Request(prompt=prompt, max_tokens=10, sampler=SamplerConfig(temperature=0.9, seed=1)))
    for _ in range(4):
        s.step()
    used = backend.cache.used_pages()
    child = s.fork(parent, sampler=SamplerConfig(temperature=0.9, seed=2), max_tokens=8)
    twin = s.fork(parent)
    assert backend.cache.used_pages() == used, "a fork takes no page until somebody writes"
    backend.cache.check_invariants()
    late = s.submit(Request(prompt=[7, 7, 7], max_tokens=2))
    cousin = s.fork(late, max_tokens=3)                       # its parent still waits: it waits right behind it
    assert [x.id for x in s.waiting] == [late, cousin]
    s.run_until_idle()
    backend.cache.check_invariants()
    assert backend.cache.free_pages() == 16 and len(backend.cache.free_slots) == backend.cache.max_requests
    p_out, c_out, t_out = (s.finished[i].tokens for i in (parent, child, twin))
    assert len(p_out) == 10 and len(c_out) == 8 and t_out == p_out[4:] and c_out[:6] != p_out[4:]
    assert s.finished[child].prompt_tokens == len(prompt) + 4
    assert len(s.finished[cousin].tokens) == 3 and s.finished[cousin].tokens[:2] == s.finished[late].tokens
    with pytest.raises(KeyError):
        s.fork(parent)                                        # it has finished
