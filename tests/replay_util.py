"""Drive ``bin/trace_run`` as a user would: a subprocess fed JSON lines, logits read back from files."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def live_tokens_needed(steps):
    """The smallest --max-tokens the trace may be given: the most tokens live requests hold at any
    time, each request's count rounded up to a multiple of 64."""
    held, away, worst = {}, {}, 0
    for st in steps:
        for parent, child in st.get("fork", []):
            held[child] = held[parent]                      # counted in full, although it shares pages at first
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], away.pop(e["id"], 0)) + len(e["tokens"])
        worst = max(worst, sum(-(-n // 64) * 64 for n in held.values()))
        for rid in st.get("preempt", []):
            away[rid] = held.pop(rid)                       # holds nothing until it returns, then everything again
        for rid in st.get("end", []):
            held.pop(rid, None)
    return worst


def run_trace(model_dir, dtype, steps, out_dir, max_tokens=None, extra=()):
    """Returns {request id: float32 [positions wanted so far, vocab]} in position order."""
    os.makedirs(out_dir, exist_ok=True)
    max_tokens = max_tokens or live_tokens_needed(steps)
    cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens), *extra]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, f"trace_run failed ({proc.returncode}):\n{proc.stderr[-4000:]}"
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps], proc.stdout[-2000:]
    with open(os.path.join(model_dir, "config.json")) as f:
        vocab = json.load(f)["vocab_size"]
    per_request, pos = {}, {}
    for st in steps:
        for parent, child in st.get("fork", []):
            pos[child] = pos[parent]
        wanted = sum(len(e.get("want", [])) for e in st["entries"])
        path = os.path.join(out_dir, f"{st['step']}.f32")
        if not wanted:
            assert not os.path.exists(path)
            for e in st["entries"]:
                pos[e["id"]] = pos.get(e["id"], 0) + len(e["tokens"])
            continue
        arr = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
        row = 0
        for e in st["entries"]:
            base = pos.get(e["id"], 0)
            for w in e.get("want", []):
                per_request.setdefault(e["id"], {})[base + w] = arr[row]
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
    return per_request


def whole(requests):
    """Each request alone and whole, one step each."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(requests.items())]


def tail_one_by_one(requests, tail=32):
    """Most of a request in one step, then its last ``tail`` tokens one by one."""
    steps, n = [], 0
    for rid, toks in requests.items():
        head = max(len(toks) - tail, 1)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        n += 1
        for i in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
            n += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def changing_portions(requests, sizes=(7, 2, 16, 3, 31, 2, 5, 17, 2, 64, 1, 2, 9)):
    """Portions of changing size, down to two tokens (and single tokens)."""
    steps, n = [], 0
    for rid, toks in requests.items():
        i, k = 0, 0
        while i < len(toks):
            c = min(sizes[k % len(sizes)], len(toks) - i)
            k += 1
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[i:i + c], "want": list(range(c))}],
                          "end": [rid] if i + c == len(toks) else []})
            i += c
            n += 1
    return steps


def mixed(requests, rng, max_live=4, prompt_frac=0.6):
    """Up to ``max_live`` requests at once: portions of some prompts beside single decoded tokens of
    others; requests are sometimes left out of a step; when one ends the next starts, so the few
    pages there are get used again."""
    queue = list(requests.items())
    live, steps, n = [], [], 0
    while queue or live:
        while queue and len(live) < max_live:
            rid, toks = queue.pop(0)
            live.append({"id": rid, "toks": toks, "at": 0, "prompt": max(2, int(len(toks) * prompt_frac))})
        entries, ended = [], []
        for r in live:
            if len(live) > 1 and rng.random() < 0.25:
                continue                                     # left out of this step, goes on later
            left = len(r["toks"]) - r["at"]
            if r["at"] < r["prompt"]:
                c = min(rng.choice([2, 3, 5, 8, 13, 21, 30]), r["prompt"] - r["at"], left)
            else:
                c = 1
            toks = r["toks"][r["at"]:r["at"] + c]
            want = list(range(c)) if rng.random() < 0.8 else []
            entries.append({"id": r["id"], "tokens": toks, "want": want})
            r["at"] += c
            if r["at"] == len(r["toks"]):
                ended.append(r["id"])
        if not entries:
            continue
        live = [r for r in live if r["id"] not in ended]
        steps.append({"step": n, "entries": entries, "end": ended})
        n += 1
    return steps


def run_steps_inprocess(engine, steps):
    """The same replay loop as bin/trace_run's (it is the same ``Replayer``), inside this process, for
    models whose parts only exist in the tests. Same result shape as ``run_trace``."""
    from glassbox_b200.engine.replay import Replayer
    rep = Replayer(engine)
    per_request, pos = {}, {}
    for st in steps:
        for parent, child in st.get("fork", []):
            pos[child] = pos[parent]
        logits = rep.run_step(st)
        arr = logits.cpu().numpy().copy() if logits is not None else None
        row = 0
        for e in st["entries"]:
            base = pos.get(e["id"], 0)
            for w in e.get("want", []):
                per_request.setdefault(e["id"], {})[base + w] = arr[row]
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
    rep.finish()
    return per_request


def forks_preemption_and_shared_prefix(vocab, rng):
    """A trace with the cache operations of a scheduler: a fork in the middle of a page (its first write copies the
    shared page), a preemption after which a newcomer takes the victim's pages before the victim returns and is
    computed again, and a request that starts on a 70-token prefix another request has already computed. Up to four
    requests are live; logits are wanted at every row. Returns (steps, {request: all its tokens})."""
    tok = lambda n: [rng.randrange(vocab) for _ in range(n)]
    prefix = tok(70)
    full = {"r0": tok(60), "r1": prefix + tok(14), "r2": prefix + tok(16), "r3": tok(56)}
    full["c0"] = full["r0"][:37] + tok(20)
    at = {"r0": 0, "r1": 0, "r2": 0, "r3": 0, "c0": 37}

    def take(rid, n, want="all"):
        toks = full[rid][at[rid]:at[rid] + n]
        assert len(toks) == n, (rid, at[rid], n)
        at[rid] += n
        return {"id": rid, "tokens": toks, "want": list(range(n)) if want == "all" else want}

    steps = [
        {"entries": [take("r0", 37)]},                                            # ends in the middle of its third page
        {"fork": [["r0", "c0"]], "entries": [take("c0", 5), take("r0", 3), take("r1", 40)]},   # both write: one copies
        {"entries": [take("r0", 1), take("c0", 1), take("r1", 30)]},             # r1 has passed the shared prefix
        {"entries": [take("r0", 1), take("c0", 1), take("r1", 2)], "preempt": ["r0"]},
        {"entries": [take("r3", 50), take("c0", 1), take("r1", 1)]},             # r3 is given the pages r0 held
        {"entries": [take("r2", 76, want=list(range(64, 76))), take("c0", 2), take("r3", 1)]},   # four live
        {"entries": [take("r3", 1), take("r2", 1), take("c0", 1), take("r1", 1)], "end": ["r1"]},
        {"entries": [take("r3", 4), take("r2", 2)], "end": ["r3"]},
        {"entries": [take("r0", 1), take("r2", 2), take("c0", 1)]},              # r0 returns: 42 tokens run again
        {"entries": [take("r0", 7), take("c0", 3)], "preempt": ["c0"]},
        {"entries": [take("r0", 1), take("r2", 1)]},
        {"entries": [take("c0", 1), take("r0", 1), take("r2", 1)]},              # c0 returns
        {"entries": [take("c0", 4), take("r0", 5), take("r2", 3)], "end": ["c0", "r0", "r2"]},
    ]
    for i, st in enumerate(steps):
        st["step"] = i
        st.setdefault("end", [])
    known = {rid: toks[:at[rid]] for rid, toks in full.items()}
    return steps, known
