"""Continuous-batching step scheduler for step-function models.

Every step is one ragged batch: each running sequence that has its prompt behind it contributes its one next token, and the
token budget that is left goes to prompt portions of the sequences still prefilling (oldest first), cut wherever the budget
ends.  Admission is bounded by the cache manager's free slots and pages.  (The reference's balance_serve scheduler hands the
model a batch of prefill chunks and decode tokens per step the same way: archive/ktransformers/server/balance_serve/
inference/forward_batch.py; its policy lives in its C++ `sched` extension.)"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional, Tuple


@dataclass
class Request:
    id: object
    prompt: List[int]
    max_new_tokens: int = 0
    output: List[int] = field(default_factory=list)
    fed: int = 0                       # prompt tokens already run
    pending: Optional[int] = None      # sampled token not yet run
    done: bool = False

    @property
    def prefilling(self) -> bool:
        return self.fed < len(self.prompt)


@dataclass
class Entry:
    request: Request
    tokens: List[int]
    want_last: bool


class Scheduler:
    def __init__(self, cache, max_step_tokens: int = 2048, max_running: Optional[int] = None, min_portion: int = 1):
        self.cache, self.max_step_tokens = cache, max_step_tokens
        self.max_running = max_running or cache.max_slots
        self.min_portion = min_portion
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []

    def add(self, req: Request) -> None:
        if not req.prompt:
            raise ValueError("empty prompt")
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def schedule(self) -> List[Entry]:
        budget, free = self.max_step_tokens, self.cache.free_tokens()
        entries: List[Entry] = []
        for r in self.running:                       # decode tokens first: they bound latency
            if not r.prefilling and r.pending is not None and budget > 0 and free >= self.cache.page_size:
                entries.append(Entry(r, [r.pending], True))
                budget -= 1
                free -= self.cache.page_size
        while self.waiting and len(self.running) < self.max_running and free >= len(self.waiting[0].prompt) + self.cache.page_size:
            free -= len(self.waiting[0].prompt) + self.cache.page_size     # admitted prompts keep their pages reserved
            self.running.append(self.waiting.popleft())
        for r in self.running:
            if r.prefilling and budget >= min(self.min_portion, len(r.prompt) - r.fed):
                n = min(budget, len(r.prompt) - r.fed)
                entries.append(Entry(r, r.prompt[r.fed:r.fed + n], r.fed + n == len(r.prompt)))
                budget -= n
        return entries

    def finish(self, req: Request) -> None:
        req.done = True
        self.running.remove(req)
        self.cache.close(req.id)
