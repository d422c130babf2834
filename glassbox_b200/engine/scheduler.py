"""Continuous batching above the step function.

Policy, after crates/glassbox-server/src/scheduler.rs:239-415:

1. *Admit* from the head of the FIFO queue while fewer than ``max_seqs`` requests run. A fresh
   request needs pages for its first portion (``min(len, token_budget)`` tokens) plus one; a
   request that was preempted before waits until its whole context plus one page fits, so it
   does not bounce. If that many pages are not free and something is running, admission stops;
   an empty engine always admits one (scheduler.rs:257-277).
2. *Plan* under the token budget: requests with one token to run (decoding) first, in running
   order, then prompt portions of ``min(remaining, budget left)`` tokens (scheduler.rs:283-298).
3. *Reserve* pages for each planned entry. **When pages run out** the most recently admitted
   request is preempted: its pages are freed, it keeps its tokens and its sampler state, goes
   back to the *front* of the queue and is recomputed later as one long prompt. If the request
   that cannot fit is the only one running, it is finished with reason "length": it is too long
   for the cache (scheduler.rs:301-330, 228-236).
4. *Run* one step: rows of every planned entry, logits wanted at the last row of each entry that
   reaches the end of its known tokens (scheduler.rs:336-352).
5. *Sample* one token per wanted row; a stop token ends the request without being emitted;
   ``max_tokens`` or ``max_position`` end it with "length" (scheduler.rs:370-404).
6. *Finish*: pages and the state slot go back to the pool (scheduler.rs:405-410, 210-226).

Sampling state (temperature, random generator) of a request that the device kernel can sample (greedy or plain
temperature) lives in the request's state slot on the device: it is written at admission, advanced by the kernel, copied
by a fork, read back when the request is preempted and written again when it returns. Requests with further filters
(top-k, top-p, min-p, repetition penalty) are sampled on the host with their ``Sampler``.

The scheduler talks to a *backend* (the ``Engine``, or a stand-in in tests) through:
``cache`` (a ``CacheManager``), ``add_request``, ``free_request``, ``reserve``, ``fork``,
``step(entries, reserve=False, sampling=flags)``, ``sample(logits, rows, samplers, contexts)``, ``set_sampling``,
``rng_state`` and ``max_position``.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence

import numpy as np

from ..sampling.sampler import Sampler, SamplerConfig

STOP, LENGTH, ABORTED = "stop", "length", "aborted"


@dataclass
class SchedulerConfig:
    token_budget: int = 256   # most tokens in one step (scheduler.rs:54-74)
    max_seqs: int = 32        # most requests running at once


@dataclass
class Request:
    prompt: Sequence[int]
    max_tokens: int = 128
    sampler: SamplerConfig = field(default_factory=SamplerConfig)
    stop: Sequence[int] = ()
    on_token: Optional[Callable[[int, int], None]] = None   # (request id, token)
    on_done: Optional[Callable[[int, str], None]] = None    # (request id, reason)


@dataclass
class Metrics:
    requests_finished: int = 0
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefix_hit_tokens: int = 0
    preemptions: int = 0
    steps: int = 0
    batch_tokens: int = 0
    ttft: List[float] = field(default_factory=list)
    itl: List[float] = field(default_factory=list)


class _Seq:
    def __init__(self, sid: int, req: Request, now: float):
        self.id = sid
        self.req = req
        self.tokens: List[int] = [int(t) for t in req.prompt]
        self.prompt_len = len(self.tokens)
        self.computed = 0
        self.sampler = Sampler(req.sampler)
        #: state of the request's random generator while it holds no state slot (before admission, after a preemption)
        self.rng_state = self.sampler.rng.state
        self.slot: Optional[int] = None
        self.device_sampled = 0 if req.sampler.needs_host else 1
        self.arrival = now
        self.first_token: Optional[float] = None
        self.last_token: Optional[float] = None
        self.admitted_before = False

    @property
    def generated(self) -> int:
        return len(self.tokens) - self.prompt_len


@dataclass
class Finished:
    tokens: List[int]
    reason: str
    prompt_tokens: int


class Scheduler:
    def __init__(self, backend, config: Optional[SchedulerConfig] = None, trace: bool = False):
        self.backend = backend
        self.config = config or SchedulerConfig()
        if self.config.token_budget <= 0 or self.config.max_seqs <= 0:
            raise ValueError("token_budget and max_seqs must be positive")
        self.waiting: Deque[_Seq] = deque()
        self.running: List[_Seq] = []
        self.next_id = 1
        self.metrics = Metrics()
        self.finished: Dict[int, Finished] = {}
        self.trace: Optional[List[dict]] = [] if trace else None
        #: launch the next pure decode step before the tokens of the running one are read (see ``_decode_step``)
        self.lookahead = True
        self._inflight = None

    # ------------------------------------------------------------------------------ requests
    def submit(self, req: Request) -> int:
        if not len(req.prompt):
            raise ValueError("a request needs at least one prompt token")
        limit = getattr(self.backend, "max_position", None)
        if limit is not None and len(req.prompt) > limit:
            # refused here, before it can fail inside a step that other requests share
            # (the reference refuses such prompts at its door too: crates/glassbox-server/src/http.rs:199-208)
            raise ValueError(f"a prompt of {len(req.prompt)} tokens is longer than the model's max_position {limit}")
        sid = self.next_id
        self.next_id += 1
        self.metrics.prompt_tokens += len(req.prompt)
        self.waiting.append(_Seq(sid, req, time.perf_counter()))
        return sid

    def is_idle(self) -> bool:
        return not self.waiting and not self.running and self._inflight is None

    def abort(self, sid: int) -> None:
        """Stop a request wherever it is; what it holds goes back to the pool
        (scheduler.rs:200-208)."""
        self._drain()
        for i, s in enumerate(self.running):
            if s.id == sid:
                del self.running[i]
                self._finish(s, ABORTED)
                return
        for s in list(self.waiting):
            if s.id == sid:
                self.waiting.remove(s)
                self._finish(s, ABORTED)
                return

    def fork(self, sid: int, sampler: Optional[SamplerConfig] = None, max_tokens: Optional[int] = None) -> int:
        """A new request that starts as a copy of request ``sid`` as it stands: everything the parent has (its
        prompt and what it generated so far) is the child's prompt, and the child shares the parent's pages until
        either writes (crates/glassbox-core/src/kv.rs:260-266). Without ``sampler`` the child takes the parent's
        sampler with its random state as it stands (it then generates what the parent generates); with one it
        goes its own way. ``max_tokens`` counts the child's own new tokens (default: what the parent has left).
        The parent must be running or waiting; a child of a waiting parent simply waits behind it."""
        import copy
        self._drain()
        parent = next((s for s in self.running if s.id == sid), None)
        waiting = next((s for s in self.waiting if s.id == sid), None) if parent is None else None
        src = parent or waiting
        if src is None:
            raise KeyError(f"request {sid} is neither running nor waiting")
        left = max(src.req.max_tokens - src.generated, 0)
        req = Request(prompt=list(src.tokens), max_tokens=left if max_tokens is None else int(max_tokens),
                      sampler=sampler or src.req.sampler, stop=src.req.stop, on_token=src.req.on_token,
                      on_done=src.req.on_done)
        cid = self.next_id
        self.next_id += 1
        child = _Seq(cid, req, time.perf_counter())
        if sampler is None:
            child.sampler = copy.deepcopy(src.sampler)
            child.rng_state = src.rng_state
        self.metrics.prompt_tokens += len(req.prompt)
        if parent is None or len(self.running) >= self.config.max_seqs or not self.backend.cache.free_slots:
            self.waiting.insert(self.waiting.index(waiting) + 1, child) if waiting is not None else self.waiting.append(child)
            return cid
        self.backend.fork(parent.id, cid)               # the slot's contents (sampling state included) are copied
        if sampler is not None:
            self._place_sampling(child)
        else:
            child.slot = self.backend.cache.slot_of(cid)
        child.computed = parent.computed
        child.admitted_before = True
        self.running.append(child)
        return cid

    def _finish(self, s: _Seq, reason: str) -> None:
        if self.backend.cache.has(s.id):
            self.backend.free_request(s.id)
        if reason != ABORTED:
            self.metrics.requests_finished += 1
            self.metrics.generated_tokens += s.generated
            if s.first_token is not None:
                self.metrics.ttft.append(s.first_token - s.arrival)
        self.finished[s.id] = Finished(tokens=s.tokens[s.prompt_len:], reason=reason, prompt_tokens=s.prompt_len)
        if s.req.on_done:
            s.req.on_done(s.id, reason)

    def _on_device(self, s: _Seq) -> bool:
        return not s.req.sampler.needs_host

    def _place_sampling(self, s: _Seq) -> None:
        """A request that has just been given a state slot: its sampling state goes there."""
        s.slot = self.backend.cache.slot_of(s.id)
        if self._on_device(s) and hasattr(self.backend, "set_sampling"):
            self.backend.set_sampling(s.id, s.req.sampler.temperature if not s.req.sampler.greedy else 0.0, s.rng_state)

    def _preempt_last(self) -> int:
        """The most recently admitted request goes back to the front of the queue (the cache library has already taken
        its pages and its slot); the state of its random generator comes back from the device with it."""
        s = self.running.pop()
        if self._on_device(s) and s.slot is not None and hasattr(self.backend, "rng_state_of_slot"):
            s.rng_state = self.backend.rng_state_of_slot(s.slot)    # the slot's contents outlive its holder until reused
        s.slot = None
        self.backend.free_request(s.id)
        s.computed = 0
        self.metrics.preemptions += 1
        self.waiting.appendleft(s)
        return s.id

    def _fits(self, span: int) -> bool:
        """Whether every cache group has the pages for ``span`` more tokens of a request plus one to grow into. A
        group that keeps a window of keys only ever holds the window and one step's rows of a request."""
        cache = self.backend.cache
        for g, group in enumerate(cache.groups):
            held = span if group.window is None else min(span, group.window + self.config.token_budget)
            if cache.free_pages(g) < cache.pages_needed(held, g) + 1:
                return False
        return True

    # ---------------------------------------------------------------------------------- step
    def _steady(self, seqs) -> bool:
        """Whether a step of exactly these requests is the steady state: nobody waits who could be admitted, and each
        brings one token that the device samples."""
        cfg = self.config
        if not seqs or len(seqs) > cfg.token_budget or (self.waiting and len(self.running) < cfg.max_seqs):
            return False
        return all(len(s.tokens) - s.computed == 1 and s.device_sampled and s.generated < s.req.max_tokens for s in seqs)

    def _decode_step(self, t0: float) -> bool:
        """The steady state: nobody can be admitted and every running request decodes one token that the device samples.
        The backend plans, runs and commits such a step in a few native calls, and the scheduler stays one step ahead of
        the device: while step t runs, step t+1 is launched for the requests that will still be running, their tokens
        taken on the device from what step t samples (who reaches ``max_tokens`` or ``max_position`` with step t is
        known beforehand; requests with stop tokens are not run ahead, since whether they stop is not). Then the
        tokens of step t are read and handed out. Returns False when the step is not of that kind (or the backend
        declines it: pages run out): the general path then takes it, from the same state."""
        launch = getattr(self.backend, "decode_launch", None)
        if launch is None:
            return False
        if self._inflight is None:
            run = list(self.running)
            if not self._steady(run):
                return False
            tokens = np.fromiter((s.tokens[-1] for s in run), dtype=np.int32, count=len(run))
            handle = launch([s.id for s in run], tokens, np.ones(len(run), dtype=np.uint8))
            if handle is None:
                return False
            self._inflight = (run, handle)
        run, handle = self._inflight
        limit = self.backend.max_position
        ahead = None
        if self.lookahead and not (self.waiting and len(self.running) < self.config.max_seqs) \
                and not any(s.req.stop for s in run):
            cont = [s for s in run if s.generated + 1 < s.req.max_tokens and len(s.tokens) + 1 < limit]
            if cont:
                h2 = launch([s.id for s in cont], None, np.ones(len(cont), dtype=np.uint8))
                if h2 is not None:
                    ahead = (cont, h2)
        self._retire(run, handle, t0)
        if ahead is not None:      # the cache learns which tokens the step that is now running was given
            cont, h2 = ahead
            self.backend.decode_commit_tokens(h2, np.fromiter((s.tokens[-1] for s in cont), dtype=np.int32, count=len(cont)))
        self._inflight = ahead
        return True

    def _retire(self, run, handle, t0: float) -> None:
        """Wait for a launched decode step and hand out its tokens."""
        picked = self.backend.decode_wait(handle)
        now = time.perf_counter()
        limit = self.backend.max_position
        done, batch_desc = [], []
        for i, s in enumerate(run):
            t = int(picked[i])
            batch_desc.append((s.id, "decode" if s.generated else "prefill", 1))
            s.computed += 1
            if s.first_token is None:
                s.first_token = now
            elif s.last_token is not None:
                self.metrics.itl.append(now - s.last_token)
            s.last_token = now
            if t in s.req.stop:
                done.append((s, STOP))
                continue
            s.tokens.append(t)
            if s.req.on_token:
                s.req.on_token(s.id, t)
            if s.generated >= s.req.max_tokens or len(s.tokens) >= limit:
                done.append((s, LENGTH))
        finished = []
        for s, reason in done:
            self.running.remove(s)
            finished.append(s.id)
            self._finish(s, reason)
        self.metrics.steps += 1
        self.metrics.batch_tokens += len(run)
        self._record(t0, batch_desc, [], finished)

    def _drain(self) -> None:
        """Bring the host level with the device: a decode step that was launched ahead is waited for and handed out."""
        if self._inflight is not None:
            run, handle = self._inflight
            self._inflight = None
            self._retire(run, handle, time.perf_counter())

    def step(self) -> bool:
        """One batch through the model. Returns False when there was nothing to do."""
        t0 = time.perf_counter()
        if self._decode_step(t0):
            return True
        self._drain()
        cfg, cache = self.config, self.backend.cache
        preempted: List[int] = []
        finished: List[int] = []

        while len(self.running) < cfg.max_seqs and self.waiting:
            s = self.waiting[0]
            span = len(s.tokens) if s.admitted_before else min(len(s.tokens), cfg.token_budget)
            if self.running and (not self._fits(span) or not cache.free_slots):
                break
            self.waiting.popleft()
            reused = self.backend.add_request(s.id, s.tokens)
            self._place_sampling(s)
            if not s.admitted_before:
                self.metrics.prefix_hit_tokens += min(reused, s.prompt_len)
            s.admitted_before = True
            s.computed = reused
            self.running.append(s)
        if not self.running:
            return False

        # Planning under the token budget (decoding requests first, then prompt portions), reserving pages, and
        # preempting the most recently admitted request when they run out, happen in the cache library in one
        # call; what is left here is to forget the preempted requests and to end a lone request that did not fit.
        remaining = [len(s.tokens) - s.computed for s in self.running]
        plan, copies, n_preempted, lone_failed = cache.plan_step([s.id for s in self.running], remaining, cfg.token_budget)
        run_copies = getattr(self.backend, "run_copies", None)
        if copies and run_copies is not None:
            run_copies(copies)
        for _ in range(n_preempted):
            preempted.append(self._preempt_last())
        if lone_failed:
            s = self.running.pop()
            finished.append(s.id)
            self._finish(s, LENGTH)
        if not plan:
            self._record(t0, [], preempted, finished)
            return not self.is_idle()

        from .engine import StepEntry
        entries, wants_for = [], []
        for i, n in plan:
            s = self.running[i]
            last = s.computed + n == len(s.tokens)
            entries.append(StepEntry(s.id, s.tokens[s.computed:s.computed + n], [n - 1] if last else []))
            if last:
                wants_for.append(i)
        done = []
        rows, samplers, contexts = [], [], []
        for j, i in enumerate(wants_for):
            s = self.running[i]
            if s.generated >= s.req.max_tokens:
                done.append((i, LENGTH))  # max_tokens 0: the prompt is read, nothing is written
                continue
            rows.append(j)
            samplers.append(s.sampler)
            contexts.append(s.tokens)
        # The device kernel samples inside the step, each row from its request's own state slot.
        sampling = None
        if rows:
            sampling = [0] * len(wants_for)
            for j, smp in zip(rows, samplers):
                sampling[j] = 0 if smp.config.needs_host else 1
        logits = self.backend.step(entries, reserve=False, sampling=sampling)

        batch_desc = []
        for i, n in plan:
            s = self.running[i]
            kind = "prefill" if (len(s.tokens) - s.computed > 1 or s.generated == 0) else "decode"
            batch_desc.append((s.id, kind, n))
            s.computed += n

        tokens = self.backend.sample(logits, rows, samplers, contexts) if rows else []
        now = time.perf_counter()
        for j, t in zip(rows, tokens):
            i = wants_for[j]
            s = self.running[i]
            if s.first_token is None:
                s.first_token = now
            elif s.last_token is not None:
                self.metrics.itl.append(now - s.last_token)
            s.last_token = now
            stop = t in s.req.stop
            if not stop:
                s.tokens.append(int(t))
                if s.req.on_token:
                    s.req.on_token(s.id, int(t))
            if stop:
                done.append((i, STOP))
            elif s.generated >= s.req.max_tokens or len(s.tokens) >= self.backend.max_position:
                done.append((i, LENGTH))
        for i, reason in sorted(done, reverse=True):
            s = self.running.pop(i)
            finished.append(s.id)
            self._finish(s, reason)
        self.metrics.steps += 1
        self.metrics.batch_tokens += sum(n for _, n in plan)
        self._record(t0, batch_desc, preempted, finished)
        return True

    def _record(self, t0, batch, preempted, finished) -> None:
        if self.trace is None:
            return
        cache = self.backend.cache
        self.trace.append({
            "step": self.metrics.steps, "ms": (time.perf_counter() - t0) * 1e3, "batch": list(batch),
            "preempted": preempted, "finished": finished, "waiting": len(self.waiting),
            "kv_used": cache.used_pages(0) if cache.groups else 0,
        })

    def run_until_idle(self, max_steps: int = 1_000_000) -> None:
        steps = 0
        while not self.is_idle():
            self.step()
            steps += 1
            if steps > max_steps:
                raise RuntimeError("the scheduler made no progress")

    def kv_utilization(self) -> float:
        cache = self.backend.cache
        return cache.used_pages(0) / cache.num_pages(0) if cache.groups else 0.0
