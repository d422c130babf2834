"""Trace replay on the GPU, through bin/trace_run as a user runs it, against the plain
implementation: each request alone and whole; most of it in one step and the last 32 tokens one by
one; portions of changing size; and mixed batches with so few pages that they are used again.
In 32-bit and in bfloat16, on tiny configurations that differ in every size and option."""
import random

import numpy as np
import pytest

from conftest import TINY, assert_logits_close
from plain.llama_plain import forward_logits
import replay_util as ru

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [70, 33, 128, 5, 90, 64, 17], "B": [100, 1, 256, 40, 64, 8, 129], "C": [300, 48, 17, 130, 65],
           "D": [320, 65, 2, 129, 200, 64]}


def make_requests(name, seed=0):
    rng = random.Random(seed)
    vocab = TINY[name]["vocab_size"]
    return {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(LENGTHS[name])}


def check(model_dir, dtype, got, requests, what, only_wanted=False):
    for rid, toks in requests.items():
        ref = forward_logits(model_dir, toks)
        have = got.get(rid, {})
        if not only_wanted:
            assert sorted(have) == list(range(len(toks))), f"{what}: {rid} is missing positions"
        if not have:
            continue
        idx = sorted(have)
        assert_logits_close(np.stack([have[i] for i in idx]), ref[idx], dtype, f"{what} {rid}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_tail_and_portions(model_dirs, tmp_path, name, dtype):
    folder = model_dirs(name, dtype)
    requests = make_requests(name)
    for label, steps in (("whole", ru.whole(requests)), ("tail", ru.tail_one_by_one(requests)),
                         ("portions", ru.changing_portions(requests))):
        got = ru.run_trace(folder, dtype, steps, str(tmp_path / label))
        check(folder, dtype, got, requests, f"{name} {label}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_mixed_batches_reuse_pages(model_dirs, sharp_dirs, tmp_path, name, dtype):
    requests = make_requests(name, seed=3)
    kinds = [("random-weights", model_dirs(name, dtype))]
    if dtype == "float32":
        kinds.append(("sharp", sharp_dirs(name, dtype)))
    for kind, folder in kinds:
        for seed in (1, 2):
            steps = ru.mixed(requests, random.Random(seed))
            assert max(len(s["entries"]) for s in steps) >= 3
            need = ru.live_tokens_needed(steps)
            assert need < sum(-(-len(t) // 64) * 64 for t in requests.values()), "pages would never be reused"
            got = ru.run_trace(folder, dtype, steps, str(tmp_path / f"{kind}{seed}"), max_tokens=need)
            check(folder, dtype, got, requests, f"{name} mixed {kind} seed {seed}", only_wanted=True)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cutting_does_not_change_logits_beyond_rounding(model_dirs, sharp_dirs, tmp_path, dtype):
    """Same model, same dtype, other ways of cutting: the difference must be rounding only, below
    the difference to the plain implementation that bfloat16 is allowed."""
    folder = sharp_dirs("B", dtype) if dtype == "float32" else model_dirs("B", dtype)
    requests = make_requests("B", seed=5)
    a = ru.run_trace(folder, dtype, ru.whole(requests), str(tmp_path / "w"))
    b = ru.run_trace(folder, dtype, ru.changing_portions(requests), str(tmp_path / "p"))
    c = ru.run_trace(folder, dtype, ru.mixed(requests, random.Random(9)), str(tmp_path / "m"))
    for rid, toks in requests.items():
        ref = np.stack([a[rid][i] for i in range(len(toks))])
        spread = ref.std()
        for other, label in ((b, "portions"), (c, "mixed")):
            idx = sorted(other.get(rid, {}))
            if not idx:
                continue
            diff = np.abs(np.stack([other[rid][i] for i in idx]) - ref[idx]).max()
            bound = 2e-5 if dtype == "float32" else 0.03 * spread
            assert diff <= bound, f"{rid} {label}: {diff:.3e} > {bound:.3e} ({dtype})"


@pytest.mark.parametrize("share", [False, True], ids=["no-sharing", "share-prefixes"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_forks_preemption_and_shared_prefixes(model_dirs, sharp_dirs, tmp_path, name, dtype, share):
    """The cache operations of a scheduler, through bin/trace_run: a fork in the middle of a page and the copy its
    first write needs, a preemption whose pages go to a newcomer before the victim returns and is computed again, a
    request that starts on a prefix another one has computed; logits at every row against the plain implementation.
    trace_run itself checks the cache's invariants at the end and that no page or slot leaked (exit code 3)."""
    kinds = [("random-weights", model_dirs(name, dtype))]
    if dtype == "float32":
        kinds.append(("sharp", sharp_dirs(name, dtype)))
    for kind, folder in kinds:
        for seed in (1, 2):
            steps, known = ru.forks_preemption_and_shared_prefix(TINY[name]["vocab_size"], random.Random(seed))
            assert max(len(s["entries"]) for s in steps) == 4
            got = ru.run_trace(folder, dtype, steps, str(tmp_path / f"{kind}{seed}"),
                               extra=("--share-prefixes",) if share else ())
            for rid, toks in known.items():
                first = {"c0": 37, "r2": 64}.get(rid, 0)     # the fork starts where its parent stood; r2 asks from 64 on
                assert sorted(got[rid]) == list(range(first, len(toks))), f"{rid} is missing positions"
            check(folder, dtype, got, known, f"{name} forks/preemption {kind} seed {seed}", only_wanted=True)
