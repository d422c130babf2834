"""The host sampler against the plain restatement, and the reference's own unit cases
(crates/glassbox-core/src/sampler.rs:188-232) (CPU)."""
import numpy as np
import pytest

from glassbox_b200.sampling import Rng, Sampler, SamplerConfig

from plain import sampler_plain


def test_rng_matches_the_plain_generator_and_repeats():
    for seed in (0, 1, 42, 2 ** 40 + 7):
        g, r = sampler_plain.xorshift64star(seed), Rng(seed)
        vals = [r.next_f32() for _ in range(50)]
        assert vals == [next(g) for _ in range(50)]
        assert all(0.0 <= v < 1.0 for v in vals)
    assert [Rng(3).next_f32() for _ in range(3)] != [Rng(4).next_f32() for _ in range(3)]


def test_filters_shape_the_distribution():
    logits = np.array([1.0, 3.0, 2.0, 0.0, -1.0], dtype=np.float32)
    d = dict(Sampler(SamplerConfig(temperature=1.0, top_k=2)).distribution(logits, []))
    assert set(d) == {1, 2} and abs(sum(d.values()) - 1) < 1e-6
    d = Sampler(SamplerConfig(temperature=1.0, top_p=0.5)).distribution(logits, [])
    assert [t for t, _ in d] == [1]                                  # the best alone already passes 0.5
    d = dict(Sampler(SamplerConfig(temperature=1.0, min_p=0.2)).distribution(logits, []))
    assert set(d) == {1, 2}                                          # e^-2 and below fall under 0.2 of the best
    d = Sampler(SamplerConfig(temperature=0.0)).distribution(logits, [])
    assert d == [(1, 1.0)]
    d = Sampler(SamplerConfig(temperature=0.0, repetition_penalty=2.0)).distribution(logits, [1])
    assert d == [(2, 1.0)]                                           # 3.0 / 2 < 2.0


def test_first_maximum_wins():
    assert Sampler(SamplerConfig()).sample(np.array([0.5, 2.0, 2.0, 1.0], dtype=np.float32), []) == 1


@pytest.mark.parametrize("cfg", [
    dict(temperature=0.8), dict(temperature=1.3, top_k=5), dict(temperature=0.7, top_p=0.9),
    dict(temperature=1.0, min_p=0.05), dict(temperature=0.9, top_k=20, top_p=0.8, min_p=0.01, repetition_penalty=1.3),
])
def test_matches_the_plain_restatement(cfg):
    rng = np.random.default_rng(5)
    logits = rng.normal(0, 2, size=97).astype(np.float32)
    context = [3, 9, 9, 40]
    ours = dict(Sampler(SamplerConfig(**cfg)).distribution(logits, context))
    theirs = sampler_plain.distribution(logits, context, **cfg)
    assert set(ours) == set(theirs)
    for t in ours:
        assert abs(ours[t] - theirs[t]) < 1e-5
    s = Sampler(SamplerConfig(seed=11, **cfg))
    g = sampler_plain.xorshift64star(11)
    misses = sum(s.sample(logits, context) != sampler_plain.draw(theirs, next(g)) for _ in range(200))
    assert misses <= 1  # float32 vs float64 cumulative sums may disagree exactly at an interval's edge
    # the empirical frequencies follow the distribution
    s = Sampler(SamplerConfig(seed=1, **cfg))
    counts = {}
    for _ in range(4000):
        t = s.sample(logits, context)
        counts[t] = counts.get(t, 0) + 1
    assert set(counts) <= set(theirs)
    top = max(theirs, key=theirs.get)
    assert abs(counts[top] / 4000 - theirs[top]) < 0.04


def test_seeded_runs_repeat():
    logits = np.random.default_rng(0).normal(size=50).astype(np.float32)
    a = [Sampler(SamplerConfig(temperature=1.0, seed=9)).sample(logits, []) for _ in range(1)]
    s1, s2 = Sampler(SamplerConfig(temperature=1.0, seed=9)), Sampler(SamplerConfig(temperature=1.0, seed=9))
    assert [s1.sample(logits, []) for _ in range(30)] == [s2.sample(logits, []) for _ in range(30)]
    assert a[0] == Sampler(SamplerConfig(temperature=1.0, seed=9)).sample(logits, [])
