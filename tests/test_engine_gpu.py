"""The engine in one process: long decoding, the first tokens of a sequence, greedy and sampled
generation through the Python entry point and the command line, the scheduler on the real engine
(batched = alone, preemption, prefix sharing, forks), and errors that must be loud."""
import random
import subprocess
import sys

import numpy as np
import pytest

from conftest import BF16_REL_MAX, ROOT, TINY, assert_logits_close
from plain import sampler_plain
from plain.llama_plain import forward_logits, greedy as plain_greedy

pytestmark = pytest.mark.gpu


def make_engine(folder, dtype, **kw):
    from glassbox_b200.engine.engine import Engine
    kw.setdefault("cache_tokens", 1024)
    kw.setdefault("max_batch_tokens", 256)
    return Engine(folder, dtype, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_first_tokens_and_long_decoding(model_dirs, name, dtype):
    from glassbox_b200.engine.engine import StepEntry
    folder = model_dirs(name, dtype)
    T = TINY[name]["max_position_embeddings"]
    toks = [random.Random(1).randrange(TINY[name]["vocab_size"]) for _ in range(T)]
    ref = forward_logits(folder, toks)
    eng = make_engine(folder, dtype)
    eng.add_request("a")
    rows = [eng.step([StepEntry("a", [t], [0])])[0].cpu().numpy() for t in toks]     # every token decoded alone
    eng.check()
    assert_logits_close(np.stack(rows[:4]), ref[:4], dtype, "first tokens")
    assert_logits_close(np.stack(rows), ref, dtype, "token by token up to max_position")
    with pytest.raises(ValueError, match="max_position"):
        eng.step([StepEntry("a", [1], [0])])


def test_warm_up_records_the_decode_graphs_before_they_are_needed(model_dirs):
    from glassbox_b200.engine.engine import StepEntry
    folder = model_dirs("A", "bfloat16")
    toks = [random.Random(3).randrange(TINY["A"]["vocab_size"]) for _ in range(40)]
    ref = forward_logits(folder, toks)
    eng = make_engine(folder, "bfloat16")
    made = eng.warm_up(max_batch=4, max_context=TINY["A"]["max_position_embeddings"])
    assert made == len(eng._graphs) and made >= 3 * 1          # batch buckets 1, 2, 4 at every table width
    assert eng.warm_up(max_batch=4, max_context=TINY["A"]["max_position_embeddings"]) == 0
    for r in ("a", "b", "c"):
        eng.add_request(r)
        eng.step([StepEntry(r, toks[:20], [])])
    rows = []
    for i in range(20, 40):                                      # three requests, then two, then one: the batch shrinks
        live = ["a", "b", "c"][:3 if i < 28 else 2 if i < 34 else 1]
        out = eng.step([StepEntry(r, [toks[i]], [0]) for r in live])
        rows.append(out[0].cpu().numpy())
    eng.check()
    decode_graphs = [k for k in eng._graphs if len(k) == 2]     # (batch bucket, table width); prompt shapes have longer keys
    assert len(decode_graphs) == made, "a decode step recorded a graph although its shape was warmed up"
    assert_logits_close(np.stack(rows), ref[20:40], "bfloat16", "decoding on warmed-up graphs")


@pytest.mark.parametrize("name, dtype, sharp", [("A", "float32", True), ("B", "float32", False), ("D", "float32", True),
                                                ("B", "bfloat16", False)])
def test_greedy_generation_through_the_entry_point(model_dirs, sharp_dirs, name, dtype, sharp):
    """Random weights of N(0, 0.02) with a tied head make a model that repeats its last prompt token whatever its
    cache holds; the tied configurations therefore run with scaled attention weights, and every case first checks
    that the expected continuation is no such echo. In bfloat16 a near-tie may fall either way: there each generated
    token must be, by the plain implementation's logits for the engine's own context, within rounding of the best."""
    import glassbox_b200
    folder = sharp_dirs(name, dtype) if sharp else model_dirs(name, dtype)
    llm = glassbox_b200.load(folder, dtype, blocks=64, budget=16, max_seqs=4)
    rng = random.Random(2)
    prompts = [[rng.randrange(TINY[name]["vocab_size"]) for _ in range(n)] for n in (5, 17, 33)]
    outs = llm.generate(prompts, 16)
    for p, out in zip(prompts, outs):
        want = plain_greedy(folder, p, 16)
        assert len(set(want)) >= 4 and want[:3] != [p[-1]] * 3, "the model echoes: the comparison would say nothing"
        if dtype == "float32":
            if out != want:   # report the margin, so a near-tie can be told from a fault
                i = next(j for j in range(16) if out[j] != want[j])
                row = np.sort(forward_logits(folder, p + want[:i])[-1])
                pytest.fail(f"greedy token {i} differs; top-2 margin there is {row[-1] - row[-2]:.3e}")
        else:
            ref = forward_logits(folder, p + out)
            for j, t in enumerate(out):
                row = ref[len(p) + j - 1]
                assert row[t] >= row.max() - BF16_REL_MAX * row.std(), \
                    f"token {j}: the engine chose {t} ({row[t]:.4f}), the best is {int(row.argmax())} ({row.max():.4f})"
            assert len(set(out)) >= 4
    single = llm.generate(prompts[0], 4)
    assert single == outs[0][:4]


def test_sampled_generation_follows_the_plain_sampler(model_dirs):
    """Tiny B, temperature 0.8, fixed per-request seeds, 24 tokens, prefill chunk 16."""
    import glassbox_b200
    folder = model_dirs("B", "float32")
    llm = glassbox_b200.load(folder, "float32", blocks=64, budget=16, max_seqs=8)
    rng = random.Random(3)
    prompts = [[rng.randrange(512) for _ in range(n)] for n in (1, 8, 40, 64, 100)]
    outs = llm.generate(prompts, 24, temperature=0.8, seed=100)
    assert outs == llm.generate(prompts, 24, temperature=0.8, seed=100), "seeded runs repeat"
    for i, (p, out) in enumerate(zip(prompts, outs)):
        uniforms = sampler_plain.xorshift64star(100 + i)
        toks = list(p)
        for j, t in enumerate(out):
            dist = sampler_plain.distribution(forward_logits(folder, toks)[-1], toks, temperature=0.8)
            r = next(uniforms)
            want = sampler_plain.draw(dist, r)
            if t != want:
                acc, lo = 0.0, None
                for tok in sorted(dist):     # a draw within 1e-5 of an interval's edge may fall either way
                    if tok in (t, want):
                        lo = acc if lo is None else lo
                    acc += dist[tok]
                    if tok in (t, want) and lo is not None and abs(acc - r) < 1e-5:
                        break
                else:
                    pytest.fail(f"request {i} token {j}: sampled {t}, the plain sampler draws {want}")
            toks.append(t)
    filtered = llm.generate(prompts[:2], 8, temperature=0.9, top_k=5, top_p=0.9, repetition_penalty=1.2, seed=4)
    assert all(len(o) == 8 for o in filtered)


class StepSpy:
    """Stands between a scheduler and the engine and keeps, for every wanted row of every step, the request, the
    position and the logits the engine returned."""

    def __init__(self, engine):
        self.engine, self.rows = engine, []
        self.real_step = engine.step
        engine.step = self.step
        engine.decode_launch = None    # (the scheduler's short cut for pure decode steps hands out tokens, not logits)

    def step(self, entries, **kw):
        starts = [self.engine.cache.length(e.request) for e in entries]
        logits = self.real_step(entries, **kw)
        host = logits.cpu().numpy().copy()
        r = 0
        for e, start in zip(entries, starts):
            for w in e.want:
                self.rows.append((e.request, start + w, host[r]))
                r += 1
        return logits


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_scheduler_on_the_engine_logits_survive_preemption_and_recomputation(model_dirs, dtype):
    """Ten requests in nine pages: requests are preempted, lose their pages to others, and are computed again (partly
    from the prefix cache). Every row of logits the scheduler sampled from, before and after a preemption, is
    compared with the plain implementation on that request's own tokens; tiny B's continuations are no echoes."""
    import glassbox_b200
    folder = model_dirs("B", dtype)
    rng = random.Random(99)
    prompts = [[rng.randrange(512) for _ in range(rng.randrange(1, 40))] for _ in range(10)]
    llm = glassbox_b200.load(folder, dtype, blocks=9, budget=64, max_seqs=8, prefix_cache=True)   # pages run out
    spy = StepSpy(llm.engine)
    ids_before = llm.scheduler.next_id
    llm.scheduler.trace = []
    outs, reasons = llm.generate(prompts, 20, return_reasons=True)
    assert llm.scheduler.metrics.preemptions > 0, "the test did not exercise preemption"
    victims = {sid for rec in llm.scheduler.trace for sid in rec["preempted"]}
    assert victims and all(r == "length" for r in reasons)     # every victim came back and ran to its 20 tokens
    llm.engine.cache.check_invariants()
    assert llm.engine.cache.free_pages() == 9
    full = {ids_before + i: p + out for i, (p, out) in enumerate(zip(prompts, outs))}
    ref = {sid: forward_logits(folder, toks) for sid, toks in full.items()}
    by_request = {}
    for sid, pos, row in spy.rows:
        by_request.setdefault(sid, []).append((pos, row))
    assert all(len(by_request[sid]) == 20 for sid in victims), "a preempted request lost or repeated a token"
    for sid, rows in by_request.items():
        got = np.stack([r for _, r in rows])
        assert_logits_close(got, ref[sid][[p for p, _ in rows]], dtype, f"request {sid} through the scheduler")
    if dtype == "float32":
        for p, out in zip(prompts, outs):
            assert out == plain_greedy(folder, p, 20)
            assert len(set(out)) >= 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_scheduler_on_the_engine_prefix_sharing_aborts_and_forks(model_dirs, dtype):
    """On the real engine: a shared 70-token prefix is found in the cache and changes no logits; aborted requests give
    everything back; a forked request continues from its parent's pages with a sampler of its own."""
    from glassbox_b200.engine.scheduler import ABORTED, Request, Scheduler, SchedulerConfig
    from glassbox_b200.sampling import SamplerConfig
    folder = model_dirs("B", dtype)
    rng = random.Random(8)
    prefix = [rng.randrange(512) for _ in range(70)]
    jobs = [prefix + [rng.randrange(512) for _ in range(rng.randrange(1, 10))] for _ in range(4)]
    rows = {}
    for share in (True, False):
        eng = make_engine(folder, dtype, share_prefixes=share, cache_tokens=1024, max_requests=8)
        spy = StepSpy(eng)
        s = Scheduler(eng, SchedulerConfig(token_budget=32, max_seqs=2))
        ids = [s.submit(Request(prompt=p, max_tokens=4)) for p in jobs]
        s.run_until_idle()
        eng.check()
        eng.cache.check_invariants()
        assert eng.cache.free_pages() == eng.cache.num_pages()
        assert (s.metrics.prefix_hit_tokens >= 64) == share
        outs = [s.finished[i].tokens for i in ids]
        for sid, pos, row in spy.rows:
            toks = jobs[ids.index(sid)] + outs[ids.index(sid)]
            rows.setdefault(share, []).append((row, forward_logits(folder, toks)[pos]))
    for share, pairs in rows.items():
        assert_logits_close(np.stack([a for a, _ in pairs]), np.stack([b for _, b in pairs]), dtype,
                            f"prefix sharing {share}")

    eng = make_engine(folder, dtype, cache_tokens=512, max_requests=8)
    s = Scheduler(eng, SchedulerConfig(token_budget=16, max_seqs=4))
    ids = [s.submit(Request(prompt=[rng.randrange(512) for _ in range(rng.randrange(1, 30))], max_tokens=12)) for _ in range(8)]
    steps = 0
    while not s.is_idle():
        s.step()
        steps += 1
        if steps % 3 == 0:
            s.abort(rng.choice(ids))
        eng.cache.check_invariants()
    eng.check()
    assert eng.cache.free_pages() == eng.cache.num_pages() and len(eng.cache.free_slots) == eng.cache.max_requests
    assert any(f.reason == ABORTED for f in s.finished.values())

    # fork through the scheduler: the child shares the parent's pages and goes its own way
    eng = make_engine(folder, dtype, cache_tokens=512, max_requests=8)
    spy = StepSpy(eng)
    s = Scheduler(eng, SchedulerConfig(token_budget=64, max_seqs=4))
    prompt = [rng.randrange(512) for _ in range(37)]
    parent = s.submit(Request(prompt=prompt, max_tokens=10, sampler=SamplerConfig(temperature=0.9, seed=1)))
    for _ in range(4):
        s.step()
    assert len(s.running[0].tokens) == 37 + 4
    child = s.fork(parent, sampler=SamplerConfig(temperature=0.9, seed=2), max_tokens=8)   # its prompt: all so far
    twin = s.fork(parent)                        # the parent's sampler state and limit: the same continuation
    s.run_until_idle()
    eng.check()
    eng.cache.check_invariants()
    assert eng.cache.free_pages() == eng.cache.num_pages()
    p_out, c_out, t_out = (s.finished[i].tokens for i in (parent, child, twin))
    assert len(p_out) == 10 and len(c_out) == 8 and c_out[:6] != p_out[4:] and t_out == p_out[4:]
    assert s.finished[child].prompt_tokens == 41
    full = {parent: prompt + p_out, child: prompt + p_out[:4] + c_out, twin: prompt + p_out}
    for sid, pos, row in spy.rows:
        assert_logits_close(row[None], forward_logits(folder, full[sid])[pos][None], dtype, f"fork: request {sid} at {pos}")


def test_prefix_sharing_and_forks_do_not_change_logits(model_dirs):
    from glassbox_b200.engine.engine import StepEntry
    folder = model_dirs("B", "float32")
    rng = random.Random(7)
    prefix = [rng.randrange(512) for _ in range(70)]
    a, b = prefix + [1, 2, 3], prefix + [9, 8, 7, 6]
    eng = make_engine(folder, "float32", share_prefixes=True, cache_tokens=256)
    assert eng.add_request("a", a) == 0
    eng.step([StepEntry("a", a, [len(a) - 1])])
    reused = eng.add_request("b", b)
    assert reused == 64
    got = eng.step([StepEntry("b", b[reused:], list(range(len(b) - reused)))]).cpu().numpy()
    assert_logits_close(got, forward_logits(folder, b)[reused:], "float32", "after a shared prefix")
    # fork: the child shares every page, writes into a copy of the partial last page
    eng.fork("a", "c")
    tail_c, tail_a = [5, 5, 5], [6, 6]
    got_c = eng.step([StepEntry("c", tail_c, [0, 1, 2])]).cpu().numpy()
    got_a = eng.step([StepEntry("a", tail_a, [0, 1])]).cpu().numpy()
    assert_logits_close(got_c, forward_logits(folder, a + tail_c)[len(a):], "float32", "forked child")
    assert_logits_close(got_a, forward_logits(folder, a + tail_a)[len(a):], "float32", "parent after fork")
    eng.cache.check_invariants()
    for r in "abc":
        eng.free_request(r)
    assert eng.cache.free_pages() == eng.cache.num_pages()


def test_bad_input_is_loud_not_wrong(model_dirs):
    from glassbox_b200.engine.engine import StepEntry
    from glassbox_b200.kernels import KernelError
    eng = make_engine(model_dirs("A", "float32"), "float32")
    eng.add_request("a")
    eng.step([StepEntry("a", [1, 2, 999], [2])])          # token id outside the vocabulary of 256
    with pytest.raises(KernelError, match="token id"):
        eng.check()
    with pytest.raises(KeyError):
        eng.step([StepEntry("nobody", [1], [0])])
    with pytest.raises(ValueError):
        eng.step([StepEntry("a", [1], [3])])


def test_command_line(model_dirs):
    folder = model_dirs("B", "float32")                 # untied head: its continuations are no echoes of the prompt
    assert len(set(plain_greedy(folder, [5, 17, 3], 6))) >= 3
    out = subprocess.run([sys.executable, "-m", "glassbox_b200", "generate", "--model", folder, "--dtype", "f32",
                          "--prompt", "5 17 3; 9,9,9,9", "-n", "6", "--blocks", "32"],
                         capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = [[int(t) for t in l.split()] for l in out.stdout.strip().splitlines()]
    assert lines == [plain_greedy(folder, [5, 17, 3], 6), plain_greedy(folder, [9, 9, 9, 9], 6)]
    assert "tok/s" in out.stderr
    bad = subprocess.run([sys.executable, "-m", "glassbox_b200", "generate"], capture_output=True, text=True, cwd=ROOT)
    assert bad.returncode == 2 and "usage" in bad.stderr


def test_sampling_state_lives_in_the_slot_and_survives_preemption(model_dirs):
    """Temperature sampling on the device from each request's own state slot: the draws of a request are those of its own
    xorshift64* generator in order, whatever else is in the batch, and a request that is preempted and computed again
    goes on with the generator where it stood (the state is read back from the slot and written into the new one)."""
    import glassbox_b200
    folder = model_dirs("B", "float32")
    rng = random.Random(21)
    prompts = [[rng.randrange(512) for _ in range(rng.randrange(5, 40))] for _ in range(8)]
    roomy = glassbox_b200.load(folder, "float32", blocks=64, budget=64, max_seqs=8)
    want = roomy.generate(prompts, 16, temperature=0.8, seed=7)
    assert roomy.scheduler.metrics.preemptions == 0
    tight = glassbox_b200.load(folder, "float32", blocks=9, budget=64, max_seqs=8)       # pages run out
    got = tight.generate(prompts, 16, temperature=0.8, seed=7)
    assert tight.scheduler.metrics.preemptions > 0, "the test did not exercise preemption"
    same = sum(a == b for a, b in zip(got, want))
    # a draw within rounding of an interval's edge may fall either way once batches differ; most requests must agree outright
    assert same >= 6, f"only {same} of 8 requests kept their random sequence over a preemption"
    for a, b in zip(got, want):
        k = next((i for i in range(16) if a[i] != b[i]), 16)
        assert k >= 1
    alone = glassbox_b200.load(folder, "float32", blocks=64, budget=64, max_seqs=1)
    for i in (0, 3):
        assert alone.generate([prompts[i]], 16, temperature=0.8, seed=7 + i)[0] == want[i]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_one_step_ahead_of_the_device_changes_nothing(model_dirs, dtype):
    """Pure decode steps are launched one ahead, their tokens taken on the device from what the step before sampled.
    Requests of different lengths and limits (so that the batch shrinks as they end), one with a stop token (which is
    not run ahead), temperature and greedy side by side, an abort and a fork in mid-flight: token for token what the
    scheduler generates when it waits for every step."""
    from glassbox_b200.engine.scheduler import Request, Scheduler, SchedulerConfig
    from glassbox_b200.sampling import SamplerConfig
    folder = model_dirs("B", dtype)
    rng = random.Random(31)
    prompts = [[rng.randrange(512) for _ in range(n)] for n in (5, 33, 17, 60, 9, 2)]
    limits = [30, 7, 19, 25, 40, 12]

    def run(lookahead, stop_for_last):
        eng = make_engine(folder, dtype, cache_tokens=1024, max_requests=8)
        s = Scheduler(eng, SchedulerConfig(token_budget=128, max_seqs=8))
        s.lookahead = lookahead
        ids = []
        for i, (p, n) in enumerate(zip(prompts, limits)):
            cfg = SamplerConfig(temperature=0.8 if i % 2 else 0.0, seed=50 + i)
            ids.append(s.submit(Request(prompt=p, max_tokens=n, sampler=cfg, stop=stop_for_last if i == len(prompts) - 1 else ())))
        steps, extra = 0, []
        while not s.is_idle():
            s.step()
            steps += 1
            if steps == 6:
                s.abort(ids[3])
                extra.append(s.fork(ids[4], max_tokens=5))
        eng.check()
        eng.cache.check_invariants()
        assert eng.cache.free_pages() == eng.cache.num_pages() and len(eng.cache.free_slots) == eng.cache.max_requests
        child = s.finished[extra[0]]
        at = child.prompt_tokens - len(prompts[4])        # how far the parent was when it was forked
        return ([s.finished[i].tokens for i in ids], [s.finished[i].reason for i in ids], child.tokens, at, eng.graph_replays)

    plain_out, plain_why, plain_child, plain_at, _ = run(False, ())
    ahead_out, ahead_why, ahead_child, ahead_at, replays = run(True, ())
    assert replays > 20 and plain_why[3] == ahead_why[3] == "aborted"
    for i in range(len(prompts)):
        if i == 3:      # aborted in mid-flight: one mode is a step further when the abort arrives; what both have must agree
            k = min(len(plain_out[3]), len(ahead_out[3]))
            assert k > 0 and plain_out[3][:k] == ahead_out[3][:k]
        else:
            assert ahead_out[i] == plain_out[i] and ahead_why[i] == plain_why[i], f"request {i}"
    # the forked twin (the parent's sampler state as it stood) generates what the parent goes on to generate, in either mode
    assert plain_child == plain_out[4][plain_at:plain_at + 5] and ahead_child == ahead_out[4][ahead_at:ahead_at + 5]
    stop_token = plain_out[5][3]                      # the last request stops at what was its fourth token
    stopped_plain = run(False, (stop_token,))
    stopped_ahead = run(True, (stop_token,))
    assert stopped_ahead[0][5] == stopped_plain[0][5] and stopped_plain[1][5] == stopped_ahead[1][5] == "stop"
    assert stopped_ahead[0][:3] == stopped_plain[0][:3]
