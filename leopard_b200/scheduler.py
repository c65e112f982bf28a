"""Request scheduler of the language-model engines: continuous batching over `engine.step`.

Requests wait in arrival order.  Each call of `Scheduler.step()` runs ONE engine step: if requests are waiting and the token budget
allows, a PREFILL step packs their whole prompts into one batch (rows of different requests are independent: the kernels take
per-row request and position tables, there is no padding); otherwise a DECODE step advances every running request by one token.  The
sampler picks the next token from the last row's logits; a request ends on an end-of-sequence id or its token limit, and its cache
pages and state slot go back to the pools at once, so a later request can take them.

The engine interface is two methods: step(entries) -> logits of the wanted rows, finish(key).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, Iterable, List, Optional, Sequence, Set

from .sampling import Sampler, SamplingParams
from .seqlm import StepEntry


@dataclass
class Request:
    key: Hashable
    prompt: Sequence[int]
    max_new_tokens: int = 16
    eos: Set[int] = field(default_factory=set)
    output: List[int] = field(default_factory=list)
    done: bool = False


class Scheduler:
    def __init__(self, engine, sampler: Optional[Sampler] = None, max_batch_tokens: int = 8192, max_running: int = 64):
        self.engine = engine
        self.sampler = sampler or Sampler(SamplingParams())
        self.max_batch_tokens = max_batch_tokens
        self.max_running = max_running
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: Dict[Hashable, Request] = {}
        self.steps = 0

    def add(self, req: Request) -> None:
        if len(req.prompt) == 0:
            raise ValueError("empty prompt")
        if req.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        self.waiting.append(req)

    def _admit(self) -> List[Request]:
        batch, tokens = [], 0
        while self.waiting and len(self.running) + len(batch) < self.max_running:
            n = len(self.waiting[0].prompt)
            if batch and tokens + n > self.max_batch_tokens:
                break
            tokens += n
            batch.append(self.waiting.popleft())
        return batch

    def step(self) -> bool:
        """One engine step; False when there is nothing left to do."""
        new = self._admit()
        if new:
            batch = new
            entries = [StepEntry(r.key, list(r.prompt), [len(r.prompt) - 1]) for r in new]
        elif self.running:
            batch = self.running
            entries = [StepEntry(r.key, [r.output[-1]], [0]) for r in batch]
        else:
            return False
        logits = self.engine.step(entries)
        ids = self.sampler(logits).tolist()          # device -> host: the stopping criterion
        self.steps += 1
        still = []
        for r, t in zip(batch, ids):
            r.output.append(int(t))
            if int(t) in r.eos or len(r.output) >= r.max_new_tokens:
                r.done = True
                self.engine.finish(r.key)
                self.finished[r.key] = r
            else:
                still.append(r)
        if new:
            self.running.extend(still)
        else:
            self.running = still
        return True

    def run(self) -> Dict[Hashable, Request]:
        while self.step():
            pass
        return self.finished


def generate(engine, prompts: Iterable[Sequence[int]], max_new_tokens: int = 16, eos: Optional[Set[int]] = None,
             sampling: Optional[SamplingParams] = None, **sched_kw) -> List[List[int]]:
    """Greedy (or sampled) continuation of every prompt through the scheduler; returns the new tokens per prompt."""
    sched = Scheduler(engine, Sampler(sampling), **sched_kw)
    reqs = [Request(key=("gen", i), prompt=list(p), max_new_tokens=max_new_tokens, eos=set(eos or ())) for i, p in enumerate(prompts)]
    for r in reqs:
        sched.add(r)
    sched.run()
    return [r.output for r in reqs]
