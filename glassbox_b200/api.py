"""The Python entry point, in Glassbox's manner: a ``Generator`` that feeds one sequence
(crates/glassbox-core/src/lib.rs:21-62), ``greedy`` (lib.rs:64-74), and ``LLM.generate`` which
submits requests to the continuous-batching scheduler and steps it until they are done
(crates/glassbox-server/src/scheduler.rs:161, 239). Text is out of scope: prompts and results are
token ids.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import numpy as np

from .engine.engine import Engine, StepEntry
from .engine.scheduler import Request, Scheduler, SchedulerConfig
from .sampling.sampler import SamplerConfig


class LLM:
    """A loaded model with its cache and scheduler.

    Option names follow the reference's command line (crates/glassbox-server/src/main.rs:322-330):
    ``blocks`` pages of 16 tokens in the cache (2048), ``budget`` tokens per step (256),
    ``max_seqs`` requests running at once (32), ``prefix_cache`` (on).
    """

    def __init__(self, model_dir: str, dtype: str = "bfloat16", *, blocks: int = 2048, budget: int = 256,
                 max_seqs: int = 32, prefix_cache: bool = True, page_size: int = 16, device: str = "cuda:0"):
        self.engine = Engine(model_dir, dtype, num_pages=blocks, page_size=page_size, max_batch_tokens=budget,
                             max_requests=max_seqs, share_prefixes=prefix_cache, device=device)
        self.scheduler_config = SchedulerConfig(token_budget=budget, max_seqs=max_seqs)
        self.scheduler = Scheduler(self.engine, self.scheduler_config)

    @property
    def config(self):
        return self.engine.config

    def warm_up(self, max_batch: Optional[int] = None, max_context: Optional[int] = None) -> int:
        """Record the CUDA graphs of decode steps up to ``max_batch`` requests and ``max_context`` tokens now,
        instead of inside the first step of each shape (a few tens of milliseconds each). Defaults: the
        scheduler's ``max_seqs`` and what the cache holds. Returns the number of graphs recorded."""
        mb = self.scheduler_config.max_seqs if max_batch is None else max_batch
        mc = min(self.engine.num_pages * self.engine.page_size, self.engine.config.max_position) if max_context is None \
            else max_context
        return self.engine.warm_up(mb, mc)

    def generate(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]], max_tokens: int = 128, *,
                 temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0,
                 repetition_penalty: float = 1.0, seed: int = 0, stop: Sequence[int] = (),
                 return_reasons: bool = False):
        """Generate up to ``max_tokens`` tokens after each prompt. ``prompts`` is one list of token
        ids or a list of such lists; request i samples with seed ``seed + i``. Returns the new
        tokens (one list, or a list of lists in the order given)."""
        single = len(prompts) > 0 and not isinstance(prompts[0], (list, tuple, np.ndarray))
        batch = [prompts] if single else list(prompts)
        limit = self.engine.max_position
        for i, p in enumerate(batch):
            if not 0 < len(p) <= limit:
                raise ValueError(f"prompt {i} has {len(p)} tokens; a prompt needs between 1 and max_position = {limit}")
        ids = []
        for i, p in enumerate(batch):
            cfg = SamplerConfig(temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p,
                                repetition_penalty=repetition_penalty, seed=seed + i)
            ids.append(self.scheduler.submit(Request(prompt=[int(t) for t in p], max_tokens=max_tokens, sampler=cfg,
                                                     stop=tuple(stop))))
        self.scheduler.run_until_idle()
        self.engine.check()
        done = [self.scheduler.finished.pop(i) for i in ids]
        outs = [d.tokens for d in done]
        if return_reasons:
            reasons = [d.reason for d in done]
            return (outs[0], reasons[0]) if single else (outs, reasons)
        return outs[0] if single else outs


    def fork(self, request_id: int, **kwargs) -> int:
        """Fork a request that is in flight (see ``Scheduler.fork``); for callers that drive
        ``llm.scheduler.submit`` / ``step`` themselves."""
        return self.scheduler.fork(request_id, **kwargs)


def load(model_dir: str, dtype: str = "bfloat16", **kwargs) -> LLM:
    return LLM(model_dir, dtype, **kwargs)


class Generator:
    """One sequence with its own request in the engine's cache: ``feed`` appends tokens and returns
    the float32 logits after the last one (lib.rs:39-50)."""
    _next = 0

    def __init__(self, engine: Engine):
        self.engine = engine
        Generator._next += 1
        self.rid = ("generator", Generator._next)
        self.engine.add_request(self.rid)
        self.tokens: List[int] = []

    def feed(self, tokens: Sequence[int]) -> np.ndarray:
        logits = self.engine.step([StepEntry(self.rid, list(tokens), [len(tokens) - 1])])
        self.tokens.extend(int(t) for t in tokens)
        return logits[0].cpu().numpy()

    def truncate(self, length: int) -> None:
        self.engine.cache.truncate(self.rid, length)
        del self.tokens[length:]

    def capacity(self) -> int:
        return self.engine.num_pages * self.engine.page_size

    def close(self) -> None:
        self.engine.free_request(self.rid)


def greedy(engine: Engine, prompt: Sequence[int], n: int) -> List[int]:
    """Greedy decode ``n`` tokens after ``prompt``, one request alone (lib.rs:64-74)."""
    g = Generator(engine)
    try:
        logits = g.feed(prompt)
        out = []
        for _ in range(n):
            t = int(np.argmax(logits))
            out.append(t)
            logits = g.feed([t])
        return out
    finally:
        g.close()
