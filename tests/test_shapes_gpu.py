"""The engine at SmolLM2 widths (few layers, so that the float64 plain implementation stays quick): the real head
counts and groups of the 135M, 360M and 1.7B configurations, head size 64, hidden sizes 576, 960 and 2048, the
49,152-token vocabulary. Each width runs in 32-bit and in bfloat16 under every way of cutting the work: each request
whole; most of it in one step and the last 32 tokens one by one; portions of changing size; mixed batches of up to
four requests with so few pages that they are used again; and a service-like mix in which many decoding requests lead
a batch that also carries prompt portions (the shape in which attention is split between the decode and the flash
kernel). Prompts are long enough for several key tiles. Logits are compared at a few hundred places per request."""
import random

import numpy as np
import pytest
import torch

import glassbox_b200
import replay_util as ru
from conftest import FP32_ATOL, assert_logits_close
from glassbox_b200.models.llama import make_llama_raw_config
from plain.llama_plain import forward_logits

pytestmark = pytest.mark.gpu

COMMON = dict(vocab_size=49152, rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=8192)
SHAPES = {
    "135m": dict(num_hidden_layers=2, hidden_size=576, num_attention_heads=9, num_key_value_heads=3,
                 intermediate_size=1536, rope_theta=100000.0, **COMMON),
    "360m": dict(num_hidden_layers=2, hidden_size=960, num_attention_heads=15, num_key_value_heads=5,
                 intermediate_size=2560, rope_theta=100000.0, **COMMON),
    "1.7b": dict(num_hidden_layers=1, hidden_size=2048, num_attention_heads=32, num_key_value_heads=32,
                 intermediate_size=8192, rope_theta=130000.0, **COMMON),
}
LENGTHS = [420, 150, 75, 33]
VOCAB = COMMON["vocab_size"]


def places(n):
    """The positions of an n-token request at which logits are compared: the first ones, both sides of every
    128-token tile edge and 16-token page edge near them, every eleventh, and the last 34."""
    keep = {0, 1, 2, 15, 16, 17}
    for edge in range(128, n, 128):
        keep.update((edge - 1, edge, edge + 1))
    keep.update(range(5, n, 11))
    keep.update(range(max(n - 34, 0), n))
    return sorted(p for p in keep if p < n)


def thin(steps, keep):
    """Ask only for the kept positions of each request."""
    pos = {}
    for st in steps:
        for parent, child in st.get("fork", []):
            pos[child] = pos[parent]
        for e in st["entries"]:
            base = pos.get(e["id"], 0)
            e["want"] = [w for w in e.get("want", []) if base + w in keep[e["id"]]]
            pos[e["id"]] = base + len(e["tokens"])
    return steps


def service_mix(small, long_ones, portion=130):
    """Many decoding requests at the head of every batch, portions of long prompts behind them (the scheduler's order)."""
    steps = [{"entries": [{"id": rid, "tokens": toks[:len(toks) - 12], "want": []} for rid, toks in small.items()], "end": []}]
    at = {rid: len(toks) - 12 for rid, toks in small.items()}
    at.update({rid: 0 for rid in long_ones})
    for k in range(12):
        entries = [{"id": rid, "tokens": [toks[at[rid]]], "want": [0]} for rid, toks in small.items()]
        for rid, toks in long_ones.items():
            if at[rid] < len(toks):
                c = min(portion + 7 * k, len(toks) - at[rid])
                entries.append({"id": rid, "tokens": toks[at[rid]:at[rid] + c], "want": list(range(c))})
        ended = []
        for e in entries:
            at[e["id"]] += len(e["tokens"])
            if at[e["id"]] == len({**small, **long_ones}[e["id"]]):
                ended.append(e["id"])
        steps.append({"entries": entries, "end": ended})
    for i, st in enumerate(steps):
        st["step"] = i
    assert all(at[r] == len(t) for r, t in {**small, **long_ones}.items())
    return steps


@pytest.fixture(scope="module")
def shape_models(tmp_path_factory):
    made = {}

    def get(shape, dtype):
        if (shape, dtype) not in made:
            folder = str(tmp_path_factory.mktemp(f"smollm2_{shape}_{dtype}"))
            store = torch.float32 if dtype == "float32" else torch.bfloat16
            glassbox_b200.write_random_model(folder, make_llama_raw_config(**SHAPES[shape]), 5, store)
            made[(shape, dtype)] = folder
        return made[(shape, dtype)]
    return get


def compare(folder, dtype, got, requests, keep, what):
    for rid, toks in requests.items():
        have = got.get(rid, {})
        rows = sorted(have)
        assert rows == [p for p in sorted(keep[rid]) if p in have] and rows, f"{what}: {rid} came back at other places than asked"
        ref = forward_logits(folder, toks, rows=rows)
        mine = np.stack([have[p] for p in rows])
        assert_logits_close(mine, ref, dtype, f"{what} {rid}")
        if dtype == "float32":      # the same greedy token everywhere, or a near-tie that the margin shows
            a, b = mine.argmax(axis=1), ref.argmax(axis=1)
            for i in np.nonzero(a != b)[0]:
                top = np.sort(ref[i])
                assert top[-1] - top[-2] <= 2 * FP32_ATOL, \
                    f"{what} {rid} position {rows[i]}: greedy token {a[i]} != {b[i]}, top-2 margin {top[-1] - top[-2]:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", ["135m", "360m", "1.7b"])
def test_smollm2_widths_under_every_schedule(shape_models, shape, dtype):
    from glassbox_b200.engine.engine import Engine
    folder = shape_models(shape, dtype)
    rng = random.Random(2)
    requests = {f"r{i}": [rng.randrange(VOCAB) for _ in range(n)] for i, n in enumerate(LENGTHS)}
    keep = {rid: set(places(len(t))) for rid, t in requests.items()}
    eng = Engine(folder, dtype, cache_tokens=1024, max_batch_tokens=1024, max_requests=8)
    for label, steps in (("whole", ru.whole(requests)), ("tail", ru.tail_one_by_one(requests)),
                         ("portions", ru.changing_portions(requests, sizes=(7, 2, 130, 3, 31, 2, 260, 17, 2, 64, 1, 129)))):
        got = ru.run_steps_inprocess(eng, thin(steps, keep))
        compare(folder, dtype, got, requests, keep, f"{shape} {label}")
    steps = thin(ru.mixed(requests, random.Random(1)), keep)
    need = ru.live_tokens_needed(steps)
    assert need < sum(-(-len(t) // 64) * 64 for t in requests.values()), "pages would never be reused"
    small = Engine(folder, dtype, cache_tokens=need, max_batch_tokens=1024, max_requests=8)
    compare(folder, dtype, ru.run_steps_inprocess(small, steps), requests, keep, f"{shape} mixed")
    assert small.cache.free_pages() == small.cache.num_pages()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", ["135m", "360m", "1.7b"])
def test_smollm2_widths_service_mix_splits_attention_between_two_kernels(shape_models, monkeypatch, shape, dtype):
    """Eighteen decoding requests lead each batch, portions of two long prompts follow: with 9, 15 or 32 heads that is
    more than 148 (row, head) pairs, so the bfloat16 step serves the leading rows with the decode kernel and the
    portions with the flash kernel, unpatched. In 32-bit one kernel takes all rows; the logits must agree either way."""
    from glassbox_b200.engine.engine import Engine
    from glassbox_b200.parts import attention
    split_calls = []
    real = attention.GqaAttention._attend_decode

    def counting(self, ctx, q, att, cache, n):
        if not ctx.decode_only:
            split_calls.append((n, ctx.n))
        return real(self, ctx, q, att, cache, n)
    monkeypatch.setattr(attention.GqaAttention, "_attend_decode", counting)
    folder = shape_models(shape, dtype)
    rng = random.Random(7)
    small = {f"s{i}": [rng.randrange(VOCAB) for _ in range(20 + 3 * i)] for i in range(18)}
    long_ones = {"L0": [rng.randrange(VOCAB) for _ in range(700)], "L1": [rng.randrange(VOCAB) for _ in range(300)]}
    requests = {**small, **long_ones}
    keep = {rid: set(places(len(t))) | set(range(len(t) - 12, len(t))) for rid, t in requests.items()}
    steps = thin(service_mix(small, long_ones), keep)
    eng = Engine(folder, dtype, cache_tokens=2560, max_batch_tokens=1024, max_requests=24)
    for rep in range(2):                       # the second pass replays the CUDA graphs the first one recorded
        got = ru.run_steps_inprocess(eng, steps)
        compare(folder, dtype, got, requests, keep, f"{shape} service mix pass {rep}")
    if dtype == "bfloat16":
        assert any(k == 18 and n > 18 for k, n in split_calls), "no batch was split between the two attention kernels"
    assert eng.cache.free_pages() == eng.cache.num_pages()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_at_the_benchmarked_context_length(tmp_path, dtype):
    """One layer at SmolLM2-135M widths: a prompt of 4,090 tokens in two portions, then ten tokens decoded one by one up
    to position 4,099, so that the decode kernels run with the split counts of a 4,096-token context (and one more
    table width); logits at the end of the prompt and at every decoded token against the plain implementation."""
    from glassbox_b200.engine.engine import Engine, StepEntry
    shape = dict(SHAPES["135m"], num_hidden_layers=1)
    folder = str(tmp_path / "m")
    glassbox_b200.write_random_model(folder, make_llama_raw_config(**shape), 9,
                                     torch.float32 if dtype == "float32" else torch.bfloat16)
    rng = random.Random(4)
    T, P = 4100, 4090
    toks = [rng.randrange(VOCAB) for _ in range(T)]
    eng = Engine(folder, dtype, cache_tokens=4352, max_batch_tokens=2048, max_requests=4)
    eng.add_request("a")
    eng.step([StepEntry("a", toks[:2048], [])])
    rows = [eng.step([StepEntry("a", toks[2048:P], [P - 2048 - 2, P - 2048 - 1])]).cpu().numpy()]
    for i in range(P, T):
        rows.append(eng.step([StepEntry("a", [toks[i]], [0])]).cpu().numpy())
    eng.check()
    at = [P - 2, P - 1] + list(range(P, T))
    assert_logits_close(np.concatenate(rows), forward_logits(folder, toks, rows=at), dtype, "decoding past position 4,090")
