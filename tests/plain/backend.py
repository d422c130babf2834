"""A CPU stand-in for the engine, for scheduler tests: the real ``CacheManager`` for the page
bookkeeping (that is what the scheduler's decisions act on) and the plain implementation for the
logits. It recomputes each request's whole sequence every step, so it has no cache to get wrong:
whatever the scheduler does to pages cannot change its outputs, only whether it runs."""
import numpy as np

from glassbox_b200.cache import CacheManager, GroupSpec

from .llama_plain import forward_logits, read_config


class PlainBackend:
    def __init__(self, model_dir, num_pages, page_size=16, max_requests=64, share_prefixes=True):
        self.model_dir = model_dir
        self.cache = CacheManager([GroupSpec(num_pages, page_size)], max_requests=max_requests,
                                  share_prefixes=share_prefixes)
        self.max_position = read_config(model_dir)["max_pos"]
        self.tokens = {}
        self.step_log = []

    def add_request(self, rid, prompt=()):
        reused = self.cache.add_request(rid, prompt)
        self.tokens[rid] = list(prompt[:reused])
        return reused

    def free_request(self, rid):
        self.cache.free_request(rid)
        self.tokens.pop(rid, None)

    def fork(self, parent, child):
        self.cache.fork(parent, child)
        self.tokens[child] = list(self.tokens[parent])

    def reserve(self, rid, n):
        self.cache.reserve(rid, n)

    def step(self, entries, reserve=True, sampling=None):
        rows = []
        self.step_log.append([(e.request, len(e.tokens), list(e.want)) for e in entries])
        for e in entries:
            if reserve:
                self.cache.reserve(e.request, len(e.tokens))
            assert self.cache.length(e.request) == len(self.tokens[e.request]), "positions must continue the cache"
            start = len(self.tokens[e.request])
            self.tokens[e.request].extend(e.tokens)
            if e.want:
                logits = forward_logits(self.model_dir, self.tokens[e.request])
                rows.extend(logits[start + w] for w in e.want)
            self.cache.commit(e.request, e.tokens)
        self.cache.check_invariants()
        if not rows:
            return np.zeros((0, 0), dtype=np.float32)
        return np.asarray(rows, dtype=np.float32).reshape(len(rows), -1)

    def sample(self, logits, rows, samplers, contexts):
        return [s.sample(logits[r], c) for r, s, c in zip(rows, samplers, contexts)]
