"""A model-free engine for scheduler tests: the runner returns one-hot logits on a token that is a
function of the request's own history, so outputs are exact and must not depend on batching,
portion sizes or preemption (the idea of the reference's tests/fakes.py:32-84)."""

from __future__ import annotations

import numpy as np

from turingserve_b200.cache import CacheManager, RunNeeds
from turingserve_b200.config import EngineConfig
from turingserve_b200.engine.engine import LLMEngine
from turingserve_b200.engine.scheduler import Scheduler
from turingserve_b200.parts.base import CacheNeed

VOCAB = 1000


def next_token(history: list[int]) -> int:
    return (sum(history[-3:]) + len(history)) % VOCAB


class FakeRunner:
    """Keeps each request's token history (what a cache holds) and answers from it."""

    def __init__(self, cache: CacheManager) -> None:
        self.cache = cache
        self.history: dict[str, list[int]] = {}
        self.steps: list[list[tuple[str, int]]] = []

    def step(self, entries):
        wanted = []
        self.steps.append([(e.cache.request_id, len(e.tokens)) for e in entries])
        for e in entries:
            self.cache.grow(e.cache, len(e.tokens))
            h = self.history.setdefault(e.cache.request_id, [])
            assert len(h) >= e.cache.num_tokens, "tokens arrive in order"
            del h[e.cache.num_tokens:]                             # after preemption the history restarts
            h.extend(e.tokens)
            for w in e.want:
                wanted.append(next_token(h[: e.cache.num_tokens + w + 1]))
            self.cache.advance(e.cache, len(e.tokens))
        if not wanted:
            return None
        out = np.zeros((len(wanted), VOCAB), dtype=np.float32)
        out[np.arange(len(wanted)), wanted] = 1.0
        return out


class FakeSampler:
    def sample(self, logits, rows):
        return np.asarray(logits).argmax(-1), np.zeros(len(rows), dtype=bool)


def make_fake_engine(num_pages=64, page=16, budget=64, max_seqs=8, max_model_len=4096, window=None,
                     watermark=0.0, eos=()):
    cache = CacheManager([RunNeeds(CacheNeed(1, 8, None), None)] +
                         ([RunNeeds(CacheNeed(1, 8, window), None)] if window else []), page, num_pages, max_seqs)
    runner = FakeRunner(cache)
    sched = Scheduler(cache, budget, max_seqs, watermark)
    cfg = EngineConfig(model="fake", max_num_seqs=max_seqs, max_num_batched_tokens=budget)
    return LLMEngine(cfg, runner, cache, sched, FakeSampler(), eos, max_model_len)


def expected_output(prompt: list[int], n: int, max_model_len: int = 4096, stop=()) -> list[int]:
    h = list(prompt)
    out = []
    while len(out) < n and len(h) < max_model_len:
        t = next_token(h)
        h.append(t)
        out.append(t)
        if t in stop:
            break
    return out
