"""Plain restatement of Glassbox's sampler (crates/glassbox-core/src/sampler.rs), written from
its formulas and sharing no code with ``glassbox_b200.sampling``.

One rule differs from the reference on purpose and is stated here because the engine's tests
compare against it: the final draw walks the kept tokens in token-id order, not in order of
probability (sampler.rs:156-163 walks the sorted candidates). The distribution is identical.
"""
import math


def xorshift64star(seed):
    """sampler.rs:36-47. Yields uniforms in [0, 1)."""
    mask = (1 << 64) - 1
    x = ((seed * 0x9E3779B97F4A7C15) & mask) | 1
    while True:
        x ^= x >> 12
        x ^= (x << 25) & mask
        x ^= x >> 27
        yield (((x * 0x2545F4914F6CDD1D) & mask) >> 40) / float(1 << 24)


def distribution(logits, context, temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.0):
    """sampler.rs:97-148 -> {token: probability}."""
    l = [float(v) for v in logits]
    if repetition_penalty != 1.0:                                   # sampler.rs:100-109
        for t in context:
            l[t] = l[t] / repetition_penalty if l[t] > 0 else l[t] * repetition_penalty
    if temperature <= 0.0:                                          # sampler.rs:110-112, 49-57
        best = 0
        for i, v in enumerate(l):
            if v > l[best]:
                best = i
        return {best: 1.0}
    l = [v / temperature for v in l]                                # sampler.rs:113-115
    k = len(l) if top_k == 0 else min(top_k, len(l))                # sampler.rs:116-117
    cand = sorted(range(len(l)), key=lambda i: (-l[i], i))[:k]
    mx = l[cand[0]]
    e = [math.exp(l[i] - mx) for i in cand]                         # sampler.rs:118-125
    z = sum(e)
    p = [v / z for v in e]
    if min_p > 0.0:                                                 # sampler.rs:126-129
        floor = p[0] * min_p
        keep = [j for j in range(len(cand)) if p[j] >= floor]
        cand, p = [cand[j] for j in keep], [p[j] for j in keep]
    if top_p < 1.0:                                                 # sampler.rs:130-141
        acc, keep = 0.0, len(cand)
        for j, v in enumerate(p):
            acc += v
            if acc >= top_p:
                keep = j + 1
                break
        cand, p = cand[:keep], p[:keep]
    total = sum(p)                                                  # sampler.rs:142-146
    return {t: v / total for t, v in zip(cand, p)}


def draw(dist, r):
    """Walk the cumulative sum in token-id order until it passes r; fall back to the last."""
    acc = 0.0
    for t in sorted(dist):
        acc += dist[t]
        if r < acc:
            return t
    return max(dist)
