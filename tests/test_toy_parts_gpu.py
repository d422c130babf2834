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


def test_a_state_mixer_decodes_on_recorded_graphs(tmp_path):
    """State slots have fixed addresses and the toy mixer reads its slot numbers on the device, so its decode steps
    are recorded and replayed like any others; its prompt portions, which walk the host's list of sequences, are not."""
    from glassbox_b200.engine.engine import Engine
    w = write_toy(str(tmp_path), RAW, seed=2)
    eng = Engine(str(tmp_path), "float32", cache_tokens=448, max_batch_tokens=256, max_requests=4)
    assert eng.device_cache.has_state and eng.model.recordable(True) and not eng.model.recordable(False)
    rng = random.Random(6)
    requests = {f"r{i}": [rng.randrange(RAW["vocab_size"]) for _ in range(n)] for i, n in enumerate([70, 45, 120])}
    want = {rid: truth(RAW, w, toks) for rid, toks in requests.items()}
    # the three requests decode side by side (a batch of three in a graph of four: one padding request), then two, then one
    steps = [{"step": 0, "entries": [{"id": r, "tokens": t[:20], "want": []} for r, t in requests.items()], "end": []}]
    for p in range(20, 120):
        live = [r for r, t in requests.items() if p < len(t)]
        steps.append({"step": len(steps), "entries": [{"id": r, "tokens": [requests[r][p]], "want": [0]} for r in live],
                      "end": [r for r in live if p == len(requests[r]) - 1]})
    got = ru.run_steps_inprocess(eng, steps)
    assert eng.graph_replays >= 90, "the decode steps of a model with state slots did not replay as graphs"
    for rid, toks in requests.items():
        assert sorted(got[rid]) == list(range(20, len(toks)))
        for p, row in got[rid].items():
            assert np.abs(row - want[rid][p]).max() <= 1e-4, f"{rid} position {p}"
    assert len(eng.cache.free_slots) == 4


def test_an_embedding_and_a_head_of_ones_own(tmp_path):
    """The embedding and the head are registered parts like the others: a model with an embedding that scales its rows
    and a head with a bias (both exist only in these tests) against the plain implementation run on the same weights
    with the scale folded into the table and the bias added afterwards."""
    from safetensors.torch import load_file, save_file
    import glassbox_b200
    from conftest import tiny_raw
    from glassbox_b200.engine.engine import Engine
    raw = tiny_raw("B")                                                  # untied head
    plain_dir, toy_dir = str(tmp_path / "plain"), str(tmp_path / "toy")
    glassbox_b200.write_random_model(plain_dir, raw, 3, torch.float32)
    tensors = load_file(os.path.join(plain_dir, "model.safetensors"))
    scale = 3.5
    bias = torch.randn(raw["vocab_size"], generator=torch.Generator().manual_seed(1))
    toy = dict(tensors)
    toy["lm_head.bias"] = bias
    os.makedirs(toy_dir)
    save_file(toy, os.path.join(toy_dir, "model.safetensors"))
    with open(os.path.join(toy_dir, "config.json"), "w") as f:
        json.dump(dict(raw, architectures=["ToyScaledForCausalLM"], embedding_scale=scale), f)
    folded = dict(tensors)
    folded["model.embed_tokens.weight"] = tensors["model.embed_tokens.weight"] * scale
    save_file(folded, os.path.join(plain_dir, "model.safetensors"))
    rng = random.Random(8)
    requests = {f"r{i}": [rng.randrange(raw["vocab_size"]) for _ in range(n)] for i, n in enumerate([60, 17, 100])}
    eng = Engine(toy_dir, "float32", cache_tokens=256, max_batch_tokens=128, max_requests=4)
    for label, steps in (("whole", ru.whole(requests)), ("tail", ru.tail_one_by_one(requests)),
                         ("mixed", ru.mixed(requests, random.Random(3)))):
        got = ru.run_steps_inprocess(eng, steps)
        for rid, toks in requests.items():
            want = lp.forward_logits(plain_dir, toks) + bias.double().numpy()
            for p, row in got.get(rid, {}).items():
                assert np.abs(row - want[p]).max() <= 1e-4, f"{label} {rid} position {p}"
    assert eng.graph_replays > 0


def test_cache_groups_are_sized_on_their_own(tmp_path):
    """``group_pages`` sizes each cache group from its spec: the toy model's attention keeps a window of 24 keys, and its
    group gets 10 pages where the engine's default would have given it 64. Requests far longer than 10 pages run, alone
    and two side by side through the scheduler, because the window gives pages back as it goes, and admission counts
    what a windowed group really holds (the window and one step's rows), not the length of the request."""
    from glassbox_b200.engine.engine import Engine
    from glassbox_b200.engine.scheduler import Request, Scheduler, SchedulerConfig
    raw = dict(RAW, window=24, max_position=320)
    w = write_toy(str(tmp_path), raw, seed=9)
    sized = []

    def pages(spec):
        sized.append(spec)
        return 10 if spec.window is not None else 40

    eng = Engine(str(tmp_path), "float32", cache_tokens=1024, max_batch_tokens=32, max_requests=3, group_pages=pages)
    assert [s.window for s in sized] == [24] and eng.cache.num_pages(0) == 10 and eng.device_cache.k[0].shape[1] == 10
    toks = [random.Random(5).randrange(raw["vocab_size"]) for _ in range(300)]
    want = truth(raw, w, toks)
    got = ru.run_steps_inprocess(eng, ru.changing_portions({"a": toks}, sizes=(9, 2, 16, 1, 30, 3)))
    assert max(np.abs(got["a"][p] - want[p]).max() for p in range(300)) <= 1e-4
    s = Scheduler(eng, SchedulerConfig(token_budget=16, max_seqs=2))
    assert s._fits(300) and not Scheduler(eng, SchedulerConfig(token_budget=512, max_seqs=2))._fits(300)
    ids = [s.submit(Request(prompt=toks[:200], max_tokens=3)), s.submit(Request(prompt=toks[50:250], max_tokens=3))]
    s.step()
    assert len(s.running) == 2
    s.run_until_idle()
    assert all(len(s.finished[i].tokens) == 3 for i in ids) and eng.cache.free_pages(0) == 10
