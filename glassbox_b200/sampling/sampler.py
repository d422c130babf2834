"""Host side of sampling: the per-request configuration, the random generator, and the full
filter pipeline for the options the device kernel does not take.

Semantics are those of crates/glassbox-core/src/sampler.rs:
* ``SamplerConfig`` fields and "off" values (sampler.rs:3-29): temperature 0 = greedy,
  top_k 0, top_p 1, min_p 0, repetition_penalty 1.
* xorshift64* (sampler.rs:31-47): state = seed * 0x9e3779b97f4a7c15 | 1; x ^= x >> 12;
  x ^= x << 25; x ^= x >> 27; r = (x * 0x2545f4914f6cdd1d) >> 40; r / 2^24.
* pipeline order (sampler.rs:97-148): repetition penalty on the context's tokens (divide a
  positive logit, multiply a negative one) -> greedy returns the first maximum -> divide by the
  temperature -> keep the top k -> softmax over the kept, maximum subtracted -> min_p floor
  relative to the best -> top_p: keep through the first cumulative >= p -> renormalise -> draw.
One deliberate difference: the draw walks the kept tokens in token-id order (on the device and
here alike), not in order of probability (sampler.rs:150-164). The distribution is the same;
which token a given random number lands on is not.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

import numpy as np

_M64 = (1 << 64) - 1


@dataclass
class SamplerConfig:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    seed: int = 0

    @property
    def greedy(self) -> bool:
        return not self.temperature > 0.0

    @property
    def needs_host(self) -> bool:
        """True when an option is set that the device kernel does not take."""
        return self.repetition_penalty != 1.0 or (not self.greedy and (
            self.top_k != 0 or self.top_p < 1.0 or self.min_p > 0.0))


class Rng:
    def __init__(self, seed: int):
        self.state = ((int(seed) * 0x9E3779B97F4A7C15) & _M64) | 1

    def next_f32(self) -> float:
        """Uniform in [0, 1) with 24 random bits."""
        x = self.state
        x ^= x >> 12
        x ^= (x << 25) & _M64
        x ^= x >> 27
        self.state = x
        return float(((x * 0x2545F4914F6CDD1D) & _M64) >> 40) / float(1 << 24)


def argmax_first(x: np.ndarray) -> int:
    return int(np.argmax(x))


class Sampler:
    def __init__(self, config: SamplerConfig):
        self.config = config
        self.rng = Rng(config.seed)

    def distribution(self, logits: np.ndarray, context: Sequence[int]) -> List[Tuple[int, float]]:
        """(token, probability) of every token that can be drawn, most likely first; greedy gives
        one entry of probability 1."""
        c = self.config
        l = np.asarray(logits, dtype=np.float32).copy()
        if c.repetition_penalty != 1.0:
            pen = np.float32(c.repetition_penalty)
            for t in context:  # once per occurrence, like the reference's loop over the context
                l[t] = l[t] / pen if l[t] > 0 else l[t] * pen
        if c.greedy:
            return [(argmax_first(l), 1.0)]
        l = l / np.float32(c.temperature)
        k = len(l) if c.top_k == 0 else min(c.top_k, len(l))
        order = np.argsort(-l, kind="stable")[:k]
        vals = l[order]
        e = np.exp(vals - vals[0], dtype=np.float32)
        p = e / e.sum(dtype=np.float32)
        keep = len(order)
        if c.min_p > 0.0:
            keep = int(np.count_nonzero(p >= p[0] * np.float32(c.min_p)))
            order, p = order[:keep], p[:keep]
        if c.top_p < 1.0:
            acc = np.cumsum(p, dtype=np.float32)
            hit = np.nonzero(acc >= np.float32(c.top_p))[0]
            keep = int(hit[0]) + 1 if hit.size else len(order)
            order, p = order[:keep], p[:keep]
        p = p / p.sum(dtype=np.float32)
        return [(int(t), float(q)) for t, q in zip(order, p)]

    def sample(self, logits: np.ndarray, context: Sequence[int]) -> int:
        dist = self.distribution(logits, context)
        if len(dist) == 1:
            return dist[0][0]
        r = self.rng.next_f32()
        acc = 0.0
        for t, p in sorted(dist):  # token-id order
            acc += p
            if r < acc:
                return t
        return max(t for t, _ in dist)

    def uniform(self) -> float:
        return self.rng.next_f32()
