"""A small continuous-batching engine on the batched decode step: admission by free rows and pages, rows that join and
leave between steps, greedy sampling (the part of scheduler.BatchEngine, scheduler.py:72-560, that drives batch.forward:
admission :180-239, the step :300-420, greedy :391, retirement :430-470).

Prompts: with prefill_chunk <= 1 every prompt token takes one decode step of its row, and a request's tokens are
exactly those it gets alone, whatever shares the batch with it. With prefill_chunk = T > 1 a step in which some row
still has two or more prompt tokens to feed runs as one ragged chunk through volundr_mlx_b200.chunk: every row brings
up to T tokens (prompt rows their next tokens, decoding rows their single next token), the rows' tokens lie one after
another without padding and are committed as they are (the reference feeds prompts in chunks through
session.prefill_iter, session.py:351-387, one request at a time). The weights are then read once per chunk
instead of once per prompt token. The chunk path's GEMMs round differently from the decode step's (within the bf16
bar), so tokens can differ from the stepwise engine at near-ties of the logits.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import torch

from . import batch as BT
from . import chunk as CH

PAGE = BT.PAGE


@dataclass
class Request:
    key: int
    prompt: list
    max_new: int
    fed: int = 0
    out: list = field(default_factory=list)

    @property
    def done(self):
        return len(self.out) >= self.max_new


class BatchEngine:
    def __init__(self, model, max_rows=16, n_pages=4096, max_pages_per_row=512, prefill_chunk=0):
        self.model = model
        self.prefill_chunk = int(prefill_chunk)
        self.chunk_steps = 0
        self.bc = model.make_cache(max_rows=max_rows, n_pages=n_pages, max_pages_per_row=max_pages_per_row)
        self.n_pages, self.max_pages_per_row = n_pages, max_pages_per_row
        self.waiting: deque = deque()
        self.running: dict = {}
        self.finished: dict = {}
        self.reserved = 0          # pages promised to the running requests (their worst case)
        self._next = 0

    def _pages(self, r: Request) -> int:
        return (len(r.prompt) + r.max_new + PAGE - 1) // PAGE

    def submit(self, prompt, max_new) -> int:
        assert len(prompt) >= 1 and max_new >= 1
        r = Request(self._next, [int(t) for t in prompt], int(max_new))
        assert self._pages(r) <= self.max_pages_per_row, "request longer than a row's page table"
        self._next += 1
        self.waiting.append(r)
        return r.key

    def _admit(self):
        join = []
        while self.waiting and len(self.running) + len(join) < self.bc.S:
            r = self.waiting[0]
            if self.reserved + self._pages(r) > self.n_pages:
                break   # first come first served: nobody overtakes a request that waits for pages
            self.waiting.popleft()
            self.reserved += self._pages(r)
            join.append(r)
        return join

    def step(self):
        """One batched step. Returns [(key, token)] for every token generated in it."""
        leave = [k for k, r in self.running.items() if r.done]
        for k in leave:
            r = self.running.pop(k)
            self.reserved -= self._pages(r)
            self.finished[k] = r
        join = self._admit()
        for r in join:
            self.running[r.key] = r
        if leave or join:
            self.bc.apply(leave=leave, join=[r.key for r in join])
        if not self.bc.B:
            return []
        rows = [self.running[k] for k in self.bc.keys]
        T = self._chunk_len(rows)
        if T > 1:
            return self._chunk_step(rows, T)
        toks = [r.prompt[r.fed] if r.fed < len(r.prompt) else r.out[-1] for r in rows]
        BT.forward(self.model, self.bc, toks)
        greedy = self.bc.greedy[: self.bc.B].tolist()   # (one small device-to-host read per step)
        produced = []
        for r, g in zip(rows, greedy):
            r.fed += 1
            if r.fed >= len(r.prompt):   # the token after the last one fed
                r.out.append(int(g))
                produced.append((r.key, int(g)))
        return produced

    def _chunk_len(self, rows) -> int:
        """Tokens a prompt row may bring to the next step: more than one only while a prompt has two or more tokens
        left (otherwise the step is a plain decode step)."""
        if self.prefill_chunk <= 1:
            return 1
        left = max(len(r.prompt) - r.fed for r in rows)
        return max(1, min(self.prefill_chunk, left))

    def _chunk_step(self, rows, T):
        """One ragged chunk: prompt rows bring up to T of their next tokens, decoding rows their one next token; the
        rows' tokens lie one after another (nothing is padded) and are committed as they are."""
        toks = [list(r.prompt[r.fed: r.fed + T]) if r.fed < len(r.prompt) else [r.out[-1]] for r in rows]
        n = [len(t) for t in toks]
        _, greedy, _ = CH.forward_chunk(self.model, self.bc, toks, write=True, logits_at=[k - 1 for k in n])
        greedy = greedy.tolist()
        self.chunk_steps += 1
        produced = []
        for b, r in enumerate(rows):
            r.fed += n[b]
            if r.fed >= len(r.prompt):
                g = int(greedy[b][0])
                r.out.append(g)
                produced.append((r.key, g))
        return produced

    def run(self, max_steps=1_000_000):
        """Steps until every submitted request has finished; returns {key: generated tokens}."""
        n = 0
        while (self.waiting or self.running) and n < max_steps:
            self.step()
            n += 1
            if all(r.done for r in self.running.values()) and not self.waiting:
                for k in list(self.running):
                    r = self.running.pop(k)
                    self.reserved -= self._pages(r)
                    self.finished[k] = r
                if self.bc.B:
                    self.bc.apply(leave=list(self.bc.keys))
        return {k: r.out for k, r in self.finished.items()}
