"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it builds the same
``Engine`` that generation uses and calls its step function with the entries it is told.
Input (standard input, one JSON object per line):

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` receives the logits at the wanted
places, in the order of the entries and of ``want``, as little-endian float32 [wanted, vocab].
After every step a line ``done <step>`` is printed and flushed. Requests named in ``end`` give
back what they hold after the step. The nearest things in Glassbox are ``Generator::feed``
(crates/glassbox-core/src/lib.rs:39-50) and the golden test's direct ``forward`` with arbitrary
wanted rows (crates/glassbox-core/tests/golden.rs:76-85).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


class Replayer:
    """Feeds trace steps to an engine. ``run_step`` returns the step's logits (a device tensor that
    the next step overwrites) or None when nothing was wanted."""

    def __init__(self, engine):
        self.engine = engine
        self.live = set()

    def run_step(self, rec: dict):
        from .engine import StepEntry
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in self.live:
                self.engine.add_request(rid)
                self.live.add(rid)
            entries.append(StepEntry(rid, e["tokens"], e.get("want", [])))
        logits = None
        if entries:
            out = self.engine.step(entries)
            logits = out if out.shape[0] else None
            self.engine.check()
        for rid in rec.get("end", []):
            self.engine.free_request(rid)
            self.live.discard(rid)
        return logits


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
    args = ap.parse_args(argv)

    from .engine import Engine
    os.makedirs(args.out, exist_ok=True)
    if 64 % args.page_size:
        print(f"trace_run: --page-size {args.page_size} must divide 64", file=sys.stderr)
        return 2
    pool_tokens = -(-args.max_tokens // 64) * 64
    engine = Engine(args.model, args.dtype, cache_tokens=pool_tokens, page_size=args.page_size,
                    max_batch_tokens=args.max_batch_tokens or max(pool_tokens, 64), max_requests=8)
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
    return 0


if __name__ == "__main__":
    sys.exit(main())
