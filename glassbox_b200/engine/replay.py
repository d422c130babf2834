"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it builds the same
``Engine`` that generation uses and calls its step function with the entries it is told.
Input (standard input, one JSON object per line):

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` receives the logits at the wanted
places, in the order of the entries and of ``want``, as little-endian float32 [wanted, vocab].
After every step a line ``done <step>`` is printed and flushed. Requests named in ``end`` give
back what they hold after the step.

Three optional fields drive the cache operations that a scheduler performs:

* ``"fork": [[parent, child], ...]``, applied before the step's entries: ``child`` starts as a copy
  of ``parent``, sharing every page it holds (crates/glassbox-core/src/kv.rs:260-266); the first
  write of either into the shared partial last page copies that page (kv.rs:161-196). The child may
  bring tokens in the same step.
* ``"preempt": [id, ...]``, applied after the step like ``end``: the request gives back everything it
  holds but is remembered (crates/glassbox-server/src/scheduler.rs:228-236). Its next entry still
  brings only its *next* tokens and ``want`` still indexes those; the replayer puts the tokens the
  request had before in front of them, so that they are computed again in that step (or, where they do
  not fit the step, in steps of their own just before it), as the scheduler recomputes a preempted
  request as one long prompt.
* with ``--share-prefixes``, a request that starts (or returns after a preemption) takes over whole
  leading pages that an earlier request with the same token prefix left in the cache
  (kv.rs:135-157), up to the page before its first wanted place: a wanted place is always computed.

The nearest things in Glassbox are ``Generator::feed`` (crates/glassbox-core/src/lib.rs:39-50) and
the golden test's direct ``forward`` with arbitrary wanted rows
(crates/glassbox-core/tests/golden.rs:76-85).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict, List

import numpy as np


class Replayer:
    """Feeds trace steps to an engine. ``run_step`` returns the step's logits (a device tensor that
    the next step overwrites) or None when nothing was wanted."""

    def __init__(self, engine):
        self.engine = engine
        self.live = set()
        self.history: Dict[object, List[int]] = {}     # tokens each request has brought so far
        self.preempted = set()
        self.reused_tokens = 0                          # tokens found in the prefix cache instead of computed
        self.recomputed_tokens = 0                      # tokens run again after a preemption

    def _admit(self, rid, tokens, want):
        """Start (or bring back) ``rid`` for an entry of ``tokens``/``want``; returns the tokens and wanted
        indices the engine has to run for it: what the request brought before and lost, then its new tokens,
        less what the prefix cache already holds."""
        before = self.history.get(rid, []) if rid in self.preempted else []
        full = list(before) + list(tokens)
        shareable = len(before) + (min(want) + 1 if want else len(tokens))
        reused = self.engine.add_request(rid, full[:shareable])
        self.live.add(rid)
        self.preempted.discard(rid)
        self.history.setdefault(rid, [])
        self.reused_tokens += reused
        self.recomputed_tokens += max(len(before) - reused, 0)
        return full[reused:], [len(before) - reused + w for w in want]

    def run_step(self, rec: dict):
        from .engine import StepEntry
        for parent, child in rec.get("fork", []):
            if parent in self.preempted:
                raise ValueError(f"step {rec.get('step')}: cannot fork {parent!r} while it is preempted")
            self.engine.fork(parent, child)
            self.live.add(child)
            self.history[child] = list(self.history[parent])
        entries, brought = [], []
        room = self.engine.max_batch_tokens - sum(len(e["tokens"]) for e in rec.get("entries", []))
        for e in rec.get("entries", []):
            rid, tokens, want = e["id"], list(e["tokens"]), list(e.get("want", []))
            run, run_want = tokens, want
            if rid not in self.live:
                run, run_want = self._admit(rid, tokens, want)
                extra = len(run) - len(tokens)
                while extra > max(room, 0):
                    # what was lost does not fit beside the step's own tokens: recompute it first, alone
                    k = min(extra - max(room, 0), self.engine.max_batch_tokens)
                    self.engine.step([StepEntry(rid, run[:k], [])])
                    run, run_want, extra = run[k:], [w - k for w in run_want], extra - k
                room -= max(extra, 0)
            entries.append(StepEntry(rid, run, run_want))
            brought.append((rid, tokens))
        logits = None
        if entries:
            out = self.engine.step(entries)
            logits = out if out.shape[0] else None
            self.engine.check()
        for rid, tokens in brought:
            self.history[rid].extend(tokens)
        for rid in rec.get("preempt", []):
            self.engine.free_request(rid)
            self.live.discard(rid)
            self.preempted.add(rid)
        for rid in rec.get("end", []):
            self.engine.free_request(rid)
            self.live.discard(rid)
            self.preempted.discard(rid)
            self.history.pop(rid, None)
        return logits

    def finish(self) -> None:
        """At the end of a trace: the cache's bookkeeping must be whole, and when no request is left every
        page and every state slot must be back in the pool. Raises AssertionError otherwise."""
        cache = self.engine.cache
        cache.check_invariants()
        if not self.live:
            for g in range(len(cache.groups)):
                assert cache.free_pages(g) == cache.num_pages(g), \
                    f"group {g}: {cache.num_pages(g) - cache.free_pages(g)} pages were not given back"
            assert len(cache.free_slots) == cache.max_requests, "state slots were not given back"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--max-batch-tokens", type=int, default=0,
                    help="most tokens in one step (default: max-tokens)")
    ap.add_argument("--share-prefixes", action="store_true",
                    help="a starting request takes over cached pages of an equal token prefix")
    args = ap.parse_args(argv)

    from .engine import Engine
    os.makedirs(args.out, exist_ok=True)
    if 64 % args.page_size:
        print(f"trace_run: --page-size {args.page_size} must divide 64", file=sys.stderr)
        return 2
    pool_tokens = -(-args.max_tokens // 64) * 64
    engine = Engine(args.model, args.dtype, cache_tokens=pool_tokens, page_size=args.page_size,
                    max_batch_tokens=args.max_batch_tokens or max(pool_tokens, 64), max_requests=8,
                    share_prefixes=args.share_prefixes)
    replayer = Replayer(engine)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        logits = replayer.run_step(rec)
        if logits is not None:
            arr = logits.detach().cpu().numpy().astype("<f4", copy=False)
            tmp = os.path.join(args.out, f".{step}.f32.tmp")
            with open(tmp, "wb") as f:
                f.write(np.ascontiguousarray(arr).tobytes())
            os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        print(f"done {step}", flush=True)
    try:
        replayer.finish()
    except AssertionError as e:
        print(f"trace_run: the cache is not whole at the end of the trace: {e}", file=sys.stderr)
        return 3
    print(f"trace_run: {engine.steps} engine steps, {replayer.reused_tokens} tokens taken from the prefix cache, "
          f"{replayer.recomputed_tokens} recomputed after preemption", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
