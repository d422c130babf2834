"""Command line in the manner of the ``glassbox`` binary (crates/glassbox-server/src/main.rs:9-80,
137-156, 322-330): the same option names with the same meanings where the reference has them.

    python -m glassbox_b200 generate --model DIR --prompt "5 17 3" [-n 128] [--dtype bf16|f32]
        [--temp T] [--top-p P] [--top-k K] [--min-p P] [--repeat-penalty R] [--seed N]
        [--blocks 2048] [--budget 256] [--max-seqs 32] [--no-prefix-cache]
    python -m glassbox_b200 random-model --config FILE --seed N --out DIR [--store bf16|f32]

Text and tokenizers are outside this engine, so ``--prompt`` takes token ids (separated by spaces
or commas; ``;`` separates several prompts, which are then batched) and the reply is printed as
token ids. ``--raw`` is accepted and changes nothing: there is no chat template to skip. The
chat, serve, anatomy, trace and spec-trace subcommands of the reference belong to its server,
visualizer and speculative decoder and are not part of this engine.
"""
from __future__ import annotations

import json
import sys
import time

USAGE = __doc__.split("\n\n")[1]


class Args:
    """``--name value`` lookup, as hand-rolled in main.rs:17-33."""

    def __init__(self, argv):
        self.argv = list(argv)

    def get(self, name, default=None):
        return self.argv[self.argv.index(name) + 1] if name in self.argv[:-1] else default

    def has(self, name):
        return name in self.argv

    def num(self, name, default, kind=float):
        v = self.get(name)
        try:
            return kind(v) if v is not None else default
        except ValueError:
            return default


def _die(msg: str) -> int:
    print(msg, file=sys.stderr)
    return 2


def _parse_prompts(text: str):
    prompts = []
    for chunk in text.split(";"):
        ids = [int(t) for t in chunk.replace(",", " ").split()]
        if ids:
            prompts.append(ids)
    return prompts


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    args = Args(argv)
    cmd = argv[0] if argv else None
    if cmd == "generate":
        model = args.get("--model")
        text = args.get("--prompt")
        if not model or text is None:
            return _die("usage:\n" + USAGE)
        try:
            prompts = _parse_prompts(text)
        except ValueError:
            return _die("--prompt takes token ids (integers separated by spaces or commas)")
        if not prompts:
            return _die("--prompt holds no token ids")
        from .api import LLM
        dtype = {"f32": "float32", "fp32": "float32", "float32": "float32"}.get(args.get("--dtype", "bf16"), "bfloat16")
        t0 = time.time()
        llm = LLM(model, dtype, blocks=args.num("--blocks", 2048, int), budget=args.num("--budget", 256, int),
                  max_seqs=args.num("--max-seqs", 32, int), prefix_cache=not args.has("--no-prefix-cache"))
        print(f"loaded {len(llm.config.layers)} layers, {llm.engine.weight_bytes() / 1e6:.0f} MB of weights in "
              f"{time.time() - t0:.1f}s", file=sys.stderr)
        n = args.num("-n", 128, int)
        t1 = time.time()
        outs = llm.generate(prompts, n, temperature=args.num("--temp", 0.0), top_p=args.num("--top-p", 1.0),
                            top_k=args.num("--top-k", 0, int), min_p=args.num("--min-p", 0.0),
                            repetition_penalty=args.num("--repeat-penalty", 1.0), seed=args.num("--seed", 0, int))
        secs = time.time() - t1
        for out in outs:
            print(" ".join(str(t) for t in out))
        total = sum(len(o) for o in outs)
        print(f"prompt {sum(len(p) for p in prompts)} tokens, generated {total} tokens: {total / secs:.1f} tok/s",
              file=sys.stderr)
        return 0
    if cmd == "random-model":
        cfg, out = args.get("--config"), args.get("--out")
        if not cfg or not out:
            return _die("usage:\n" + USAGE)
        import torch
        from .weights.random_init import write_random_model
        with open(cfg) as f:
            raw = json.load(f)
        store = torch.float32 if args.get("--store", "bf16") in ("f32", "fp32", "float32") else torch.bfloat16
        write_random_model(out, raw, args.num("--seed", 0, int), store)
        print(out)
        return 0
    return _die("usage:\n" + USAGE)
