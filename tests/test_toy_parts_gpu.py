"""(c)'s generality, shown with parts that exist only in these tests: a mixer with state of its own
is registered, built and stepped without a change to the framework's files; one model mixes two
kinds of mixer; the execution order names a layer twice and lets a run read another run's cache; a
feed-forward that routes tokens to experts and a position encoding that is not a rotation sit in one
model beside the framework's own parts."""
import json
import os
import random

import numpy as np
import pytest
import torch

import replay_util as ru
import toy_arch  # noqa: F401  (registers the toy parts and architectures)
from plain import llama_plain as lp

pytestmark = pytest.mark.gpu

RAW = {"architectures": ["ToyStateForCausalLM"], "vocab_size": 131, "hidden_size": 48, "num_heads": 3,
       "num_kv_heads": 3, "head_dim": 16, "intermediate_size": 72, "eps": 2e-6, "rope_theta": 5000.0,
       "max_position": 160, "decay": 0.75}


def write_toy(folder, raw, seed=0):
    from glassbox_b200.weights import write_safetensors
    g = torch.Generator().manual_seed(seed)
    d, inter, qd = raw["hidden_size"], raw["intermediate_size"], raw["num_heads"] * raw["head_dim"]
    kvd = raw["num_kv_heads"] * raw["head_dim"]
    mat = lambda r, c, s=0.08: torch.randn(r, c, generator=g) * s
    t = {"embed": mat(raw["vocab_size"], d, 0.5), "final_norm": 1 + 0.05 * torch.randn(d, generator=g),
         "state_w": mat(d, d), "wq": mat(qd, d), "wk": mat(kvd, d), "wv": mat(kvd, d), "wo": mat(d, qd)}
    for i in (0, 1):
        t[f"norm{i}a"] = 1 + 0.05 * torch.randn(d, generator=g)
        t[f"norm{i}b"] = 1 + 0.05 * torch.randn(d, generator=g)
        t[f"gate{i}"], t[f"up{i}"], t[f"down{i}"] = mat(inter, d), mat(inter, d), mat(d, inter)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), t)
    return {k: v.double().numpy() for k, v in t.items()}


def truth(raw, w, tokens):
    """The toy model from the plain parts, whole sequence, float64."""
    T, d, hd, nh, nkv = len(tokens), raw["hidden_size"], raw["head_dim"], raw["num_heads"], raw["num_kv_heads"]
    x = w["embed"][np.asarray(tokens)]
    cos, sin = lp.rope_angles(np.arange(T), hd, raw["rope_theta"])
    caches = {}
    for layer, cache, writes in raw.get("schedule", [(0, 0, True), (1, 1, True)]):
        h = lp.rms_norm(x, w[f"norm{layer}a"], raw["eps"])
        if layer == 0:
            s, out = np.zeros(d), np.zeros((T, d))
            for t in range(T):
                s = raw["decay"] * s + h[t]
                out[t] = w["state_w"] @ s
            x = x + out
        else:
            q = lp.rope((h @ w["wq"].T).reshape(T, nh, hd), cos, sin)
            if writes:
                caches[cache] = (lp.rope((h @ w["wk"].T).reshape(T, nkv, hd), cos, sin), (h @ w["wv"].T).reshape(T, nkv, hd))
            k, v = caches[cache]
            x = x + lp.attention(q, k, v, hd ** -0.5, raw.get("window")).reshape(T, nh * hd) @ w["wo"].T
        h = lp.rms_norm(x, w[f"norm{layer}b"], raw["eps"])
        x = x + lp.swiglu(h @ w[f"gate{layer}"].T, h @ w[f"up{layer}"].T) @ w[f"down{layer}"].T
    return lp.rms_norm(x, w["final_norm"], raw["eps"]) @ w["embed"].T


@pytest.mark.parametrize("schedule", [None, [(0, 0, True), (1, 1, True), (0, 2, True), (1, 1, False)]])
def test_state_mixer_is_registered_built_and_stepped(tmp_path, schedule):
    from glassbox_b200.engine.engine import Engine
    raw = dict(RAW)
    if schedule:
        raw["schedule"] = schedule      # layer 0 and layer 1 run twice; the last run reads cache layer 1
    w = write_toy(str(tmp_path), raw)
    eng = Engine(str(tmp_path), "float32", cache_tokens=448, max_batch_tokens=256, max_requests=4)
    assert eng.device_cache.has_state and not eng.cache.share_prefixes
    rng = random.Random(3)
    requests = {f"r{i}": [rng.randrange(raw["vocab_size"]) for _ in range(n)] for i, n in enumerate([90, 33, 150, 64, 7])}
    want = {rid: truth(raw, w, toks) for rid, toks in requests.items()}
    for label, steps in (("whole", ru.whole(requests)), ("tail", ru.tail_one_by_one(requests)),
                         ("portions", ru.changing_portions(requests)), ("mixed", ru.mixed(requests, random.Random(1)))):
        got = ru.run_steps_inprocess(eng, steps)
        for rid in requests:
            for p, row in got.get(rid, {}).items():
                assert np.abs(row - want[rid][p]).max() <= 1e-4, f"{label} {rid} position {p}"
    assert len(eng.cache.free_slots) == 4 and eng.cache.free_pages() == eng.cache.num_pages()


def test_a_windowed_layer_gives_pages_back_while_it_runs(tmp_path):
    from glassbox_b200.engine.engine import Engine
    raw = dict(RAW, window=24, max_position=160)
    w = write_toy(str(tmp_path), raw, seed=4)
    eng = Engine(str(tmp_path), "float32", cache_tokens=64, max_batch_tokens=64, max_requests=2)   # 4 pages only
    toks = [random.Random(5).randrange(raw["vocab_size"]) for _ in range(150)]
    want = truth(raw, w, toks)
    got = ru.run_steps_inprocess(eng, ru.changing_portions({"a": toks}, sizes=(9, 2, 16, 1, 30, 3)))
    assert sorted(got["a"]) == list(range(150))
    assert max(np.abs(got["a"][p] - want[p]).max() for p in range(150)) <= 1e-4


ROUTED = {"architectures": ["ToyRoutedForCausalLM"], "vocab_size": 149, "hidden_size": 40, "num_heads": 2,
          "num_kv_heads": 1, "head_dim": 16, "intermediate_size": 56, "eps": 1e-5, "rope_theta": 20000.0,
          "max_position": 144, "num_experts": 5, "top_k": 2, "expert_size": 24}


def write_routed(folder, raw, seed=0):
    from glassbox_b200.weights import write_safetensors
    g = torch.Generator().manual_seed(seed)
    d, hd, inter = raw["hidden_size"], raw["head_dim"], raw["intermediate_size"]
    qd, kvd, e, ei = raw["num_heads"] * hd, raw["num_kv_heads"] * hd, raw["num_experts"], raw["expert_size"]
    mat = lambda *shape, s=0.1: torch.randn(*shape, generator=g) * s
    t = {"embed": mat(raw["vocab_size"], d, s=0.5), "final_norm": 1 + 0.05 * torch.randn(d, generator=g),
         "offsets": mat(raw["max_position"], hd, s=0.3), "router": mat(e, d, s=1.0),
         "experts_gate_up": mat(e, 2 * ei, d), "experts_down": mat(e, d, ei),
         "gate": mat(inter, d), "up": mat(inter, d), "down": mat(d, inter)}
    for i in (0, 1):
        t[f"wq{i}"], t[f"wk{i}"], t[f"wv{i}"], t[f"wo{i}"] = mat(qd, d), mat(kvd, d), mat(kvd, d), mat(d, qd)
        t[f"norm{i}a"] = 1 + 0.05 * torch.randn(d, generator=g)
        t[f"norm{i}b"] = 1 + 0.05 * torch.randn(d, generator=g)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), t)
    return {k: v.double().numpy() for k, v in t.items()}


def routed_truth(raw, w, tokens):
    """The routed toy model from the plain parts, whole sequence, float64."""
    T, hd, nh, nkv = len(tokens), raw["head_dim"], raw["num_heads"], raw["num_kv_heads"]
    x = w["embed"][np.asarray(tokens)]
    cos, sin = lp.rope_angles(np.arange(T), hd, raw["rope_theta"])
    for layer in (0, 1):
        h = lp.rms_norm(x, w[f"norm{layer}a"], raw["eps"])
        q = (h @ w[f"wq{layer}"].T).reshape(T, nh, hd)
        k = (h @ w[f"wk{layer}"].T).reshape(T, nkv, hd)
        v = (h @ w[f"wv{layer}"].T).reshape(T, nkv, hd)
        if layer == 0:
            q, k = q + w["offsets"][:T, None, :], k + w["offsets"][:T, None, :]
        else:
            q, k = lp.rope(q, cos, sin), lp.rope(k, cos, sin)
        x = x + lp.attention(q, k, v, hd ** -0.5, None).reshape(T, nh * hd) @ w[f"wo{layer}"].T
        h = lp.rms_norm(x, w[f"norm{layer}b"], raw["eps"])
        if layer == 0:
            logits = h @ w["router"].T
            out = np.zeros_like(x)
            for t in range(T):
                best = np.argsort(-logits[t], kind="stable")[:raw["top_k"]]
                z = np.exp(logits[t, best] - logits[t, best].max())
                for e, p in zip(best, z / z.sum()):
                    gu = w["experts_gate_up"][e] @ h[t]
                    i = raw["expert_size"]
                    out[t] += p * (w["experts_down"][e] @ lp.swiglu(gu[:i], gu[i:]))
            x = x + out
        else:
            x = x + lp.swiglu(h @ w["gate"].T, h @ w["up"].T) @ w["down"].T
    return lp.rms_norm(x, w["final_norm"], raw["eps"]) @ w["embed"].T


def test_routed_feed_forward_and_a_learned_position_encoding_beside_the_stock_parts(tmp_path):
    from glassbox_b200.engine.engine import Engine
    w = write_routed(str(tmp_path), ROUTED)
    eng = Engine(str(tmp_path), "float32", cache_tokens=320, max_batch_tokens=160, max_requests=4)
    assert len(eng.device_cache.group_specs) == 1 and not eng.device_cache.has_state   # both layers keep keys alike
    rng = random.Random(7)
    requests = {f"r{i}": [rng.randrange(ROUTED["vocab_size"]) for _ in range(n)] for i, n in enumerate([80, 37, 140, 5])}
    want = {rid: routed_truth(ROUTED, w, toks) for rid, toks in requests.items()}
    for label, steps in (("whole", ru.whole(requests)), ("tail", ru.tail_one_by_one(requests)),
                         ("portions", ru.changing_portions(requests)), ("mixed", ru.mixed(requests, random.Random(2)))):
        got = ru.run_steps_inprocess(eng, steps)
        for rid in requests:
            for p, row in got.get(rid, {}).items():
                assert np.abs(row - want[rid][p]).max() <= 1e-4, f"{label} {rid} position {p}"
    assert eng.graph_replays > 0, "steps of these parts replay as CUDA graphs like any others"
    assert eng.cache.free_pages() == eng.cache.num_pages()
