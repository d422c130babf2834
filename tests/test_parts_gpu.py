"""Each part of a layer alone: a model in which one part is real and every other part is an identity
or adds nothing, so that the logits are that part's output; compared with the plain function of the
same part (tests/plain/llama_plain.py), in float32 and bfloat16, whole and cut into portions and
single tokens. Sizes differ from the tiny models' (odd widths, other head shapes)."""
import json
import os
import random

import numpy as np
import pytest
import torch

import replay_util as ru
import toy_arch  # noqa: F401
from plain import llama_plain as lp

pytestmark = pytest.mark.gpu

ATOL = {"float32": 2e-5, "bfloat16": 3e-2}


def build(folder, raw, tensors, dtype):
    from glassbox_b200.engine.engine import Engine
    from glassbox_b200.weights import write_safetensors
    os.makedirs(folder, exist_ok=True)
    raw = dict(raw, architectures=["OnePartForCausalLM"])
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    stored = {k: v.to(store) for k, v in tensors.items()}
    write_safetensors(os.path.join(folder, "model.safetensors"), stored)
    eng = Engine(folder, dtype, cache_tokens=1024, max_batch_tokens=512, max_requests=8)
    return eng, {k: v.double().numpy() for k, v in stored.items()}      # the values the engine really holds


def run_all_ways(eng, requests):
    outs = {}
    for label, steps in (("whole", ru.whole(requests)), ("tail", ru.tail_one_by_one(requests, tail=9)),
                         ("portions", ru.changing_portions(requests, sizes=(5, 2, 11, 1, 3, 40)))):
        outs[label] = ru.run_steps_inprocess(eng, steps)
    return outs


def check(outs, requests, truth_fn, dtype, d):
    for label, got in outs.items():
        for rid, toks in requests.items():
            want = truth_fn(toks)
            have = np.stack([got[rid][p][:d] for p in range(len(toks))])
            scale = max(1.0, np.abs(want).max())
            assert np.abs(have - want).max() <= ATOL[dtype] * scale, f"{label} {rid}: off by {np.abs(have - want).max():.3e}"


def inputs(vocab, d, seed, spread=1.0):
    g = torch.Generator().manual_seed(seed)
    embed = torch.randn(vocab, d, generator=g) * spread
    head = torch.zeros(vocab, d)
    head[:d] = torch.eye(d)
    return g, embed, head


def make_requests(vocab, lengths, seed=0):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d, eps", [(40, 1e-5), (136, 3e-6)])
def test_norm_alone(tmp_path, dtype, d, eps):
    vocab = 150
    g, embed, head = inputs(vocab, d, 1, spread=3.0)
    gain = 1 + 0.2 * torch.randn(d, generator=g)
    eng, w = build(str(tmp_path), {"part": "norm", "vocab_size": vocab, "hidden_size": d, "max_position": 128, "eps": eps},
                   {"embed": embed, "head": head, "norm": gain}, dtype)
    requests = make_requests(vocab, [70, 3, 33])
    check(run_all_ways(eng, requests), requests, lambda t: lp.rms_norm(w["embed"][t], w["norm"], eps), dtype, d)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d, inter", [(40, 56), (96, 176)])
def test_feed_forward_alone(tmp_path, dtype, d, inter):
    vocab = 150
    g, embed, head = inputs(vocab, d, 2)
    t = {"embed": embed, "head": head, "gate": torch.randn(inter, d, generator=g) * 0.3,
         "up": torch.randn(inter, d, generator=g) * 0.3, "down": torch.randn(d, inter, generator=g) * 0.3}
    eng, w = build(str(tmp_path), {"part": "ffn", "vocab_size": vocab, "hidden_size": d, "max_position": 128,
                                   "intermediate_size": inter}, t, dtype)
    requests = make_requests(vocab, [70, 3, 33])

    def truth(toks):
        x = w["embed"][toks]
        return x + lp.swiglu(x @ w["gate"].T, x @ w["up"].T) @ w["down"].T
    check(run_all_ways(eng, requests), requests, truth, dtype, d)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh, nkv, hd, theta, window", [(3, 1, 16, None, None), (4, 2, 32, 10000.0, None),
                                                       (2, 2, 64, 500000.0, 29), (6, 2, 64, None, None)])
def test_mixer_and_position_alone(tmp_path, dtype, nh, nkv, hd, theta, window):
    """Attention with and without rotary encoding, with and without a window, against the plain
    attention and rope functions."""
    d, vocab = 72 if hd < 64 else 136, 200
    g, embed, head = inputs(vocab, d, 3)
    t = {"embed": embed, "head": head, "wq": torch.randn(nh * hd, d, generator=g) * 0.25,
         "wk": torch.randn(nkv * hd, d, generator=g) * 0.25, "wv": torch.randn(nkv * hd, d, generator=g) * 0.25,
         "wo": torch.randn(d, nh * hd, generator=g) * 0.1}
    raw = {"part": "mixer", "vocab_size": vocab, "hidden_size": d, "max_position": 256, "num_heads": nh,
           "num_kv_heads": nkv, "head_dim": hd, "rope_theta": theta, "window": window}
    eng, w = build(str(tmp_path), raw, t, dtype)
    requests = make_requests(vocab, [200, 17, 65])

    def truth(toks):
        T = len(toks)
        x = w["embed"][toks]
        q = (x @ w["wq"].T).reshape(T, nh, hd)
        k = (x @ w["wk"].T).reshape(T, nkv, hd)
        v = (x @ w["wv"].T).reshape(T, nkv, hd)
        if theta is not None:
            cos, sin = lp.rope_angles(np.arange(T), hd, float(np.float32(theta)))
            q, k = lp.rope(q, cos, sin), lp.rope(k, cos, sin)
        return x + lp.attention(q, k, v, hd ** -0.5, window).reshape(T, nh * hd) @ w["wo"].T
    check(run_all_ways(eng, requests), requests, truth, dtype, d)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_arrangement_alone(tmp_path, dtype):
    """The pre-norm wiring: x += mixer(norm(x)); x += ffn(norm(x)), with real norms, attention and feed-forward."""
    d, vocab, nh, nkv, hd, inter, eps, theta = 48, 120, 3, 3, 16, 80, 2e-6, 20000.0
    g, embed, head = inputs(vocab, d, 4)
    t = {"embed": embed, "head": head, "wq": torch.randn(nh * hd, d, generator=g) * 0.2,
         "wk": torch.randn(nkv * hd, d, generator=g) * 0.2, "wv": torch.randn(nkv * hd, d, generator=g) * 0.2,
         "wo": torch.randn(d, nh * hd, generator=g) * 0.1, "gate": torch.randn(inter, d, generator=g) * 0.2,
         "up": torch.randn(inter, d, generator=g) * 0.2, "down": torch.randn(d, inter, generator=g) * 0.2,
         "norm_a": 1 + 0.2 * torch.randn(d, generator=g), "norm_b": 1 + 0.2 * torch.randn(d, generator=g)}
    raw = {"part": "block", "vocab_size": vocab, "hidden_size": d, "max_position": 128, "num_heads": nh,
           "num_kv_heads": nkv, "head_dim": hd, "rope_theta": theta, "intermediate_size": inter, "eps": eps}
    eng, w = build(str(tmp_path), raw, t, dtype)
    requests = make_requests(vocab, [100, 9])

    def truth(toks):
        T = len(toks)
        x = w["embed"][toks]
        h = lp.rms_norm(x, w["norm_a"], eps)
        cos, sin = lp.rope_angles(np.arange(T), hd, theta)
        q = lp.rope((h @ w["wq"].T).reshape(T, nh, hd), cos, sin)
        k = lp.rope((h @ w["wk"].T).reshape(T, nkv, hd), cos, sin)
        v = (h @ w["wv"].T).reshape(T, nkv, hd)
        x = x + lp.attention(q, k, v, hd ** -0.5).reshape(T, nh * hd) @ w["wo"].T
        h = lp.rms_norm(x, w["norm_b"], eps)
        return x + lp.swiglu(h @ w["gate"].T, h @ w["up"].T) @ w["down"].T
    check(run_all_ways(eng, requests), requests, truth, dtype, d)


def test_a_part_of_an_unknown_kind_is_refused():
    from glassbox_b200.parts import build_part
    with pytest.raises(ValueError, match="no mixer part registered"):
        build_part("mixer", "no_such_mixer", hidden_size=8)
