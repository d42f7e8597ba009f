"""A continuous-batching engine on the batched decode step: admission by free rows and pages, rows that join and
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

With slice_ms > 0 (and prefill_chunk = T) prompts are fed the reference's way (scheduler.py:241-263, session.prefill_iter,
session.py:351-387): the oldest admitted request is prefilled on a one-row cache of its own, chunk after chunk of T
tokens, and the chunk pass hands control back after every layer (chunk.forward_chunk_iter); while any request is
decoding, a tick spends at most slice_ms on prefill layers, stops at the next layer boundary, runs ONE decode step for
all decoding rows and picks the chunk up where it stopped in the next tick. A long prompt therefore never stalls the
decoding streams for longer than a slice plus one layer of a chunk. A request whose prompt is through moves into the
decode batch as a session.State (capture_row on the prefill cache, apply(join=[(key, state)]) on the batch).

With a session.SessionCache (sessions=...) a request resumes from the longest snapshot whose tokens are a prefix of
its prompt (its own session first), prefills only the rest, and leaves snapshots behind: at interval positions of a
long prefill, at the end of its prompt (with the logits that pick the first token) and at the end of its reply
(scheduler.py:134-190, :504-560).

With spec=True (sliced mode) a step of 1..bspec_max decoding rows is a batched speculative step (scheduler.py:432-503):
each row drafts up to T - 1 tokens by copying from its own context (volundr_mlx_b200.lookup, or any object with
propose / record / reset given as drafter_factory), all rows' [bonus, drafts] go through ONE verify pass
(batch_spec.verify_forward), each row keeps its longest accepted run plus the model's own next token
(batch_spec.commit with its count). Rows that have nothing to propose ride along; a step in which no row proposes
anything is a plain decode step.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field

import torch

from . import batch as BT
from . import batch_spec as SP
from . import chunk as CH
from .lookup import Lookup

PAGE = BT.PAGE


@dataclass
class Request:
    key: int
    prompt: list
    max_new: int
    fed: int = 0
    out: list = field(default_factory=list)
    session: object = None
    points: list = field(default_factory=list)      # snapshot positions still ahead inside the prompt
    resumed: int = 0                                # prompt tokens taken from a snapshot
    drafter: object = None                          # the row's drafter (speculative steps)
    drafter_len: int = -1                           # len(out) the drafter's history corresponds to

    @property
    def done(self):
        return len(self.out) >= self.max_new


class BatchEngine:
    def __init__(self, model, max_rows=16, n_pages=4096, max_pages_per_row=512, prefill_chunk=0, slice_ms=0.0, sessions=None,
                 clock=time.perf_counter, spec=False, spec_T=8, bspec_max=4, bspec_rows=16, drafter_factory=Lookup):
        self.model = model
        self.prefill_chunk = int(prefill_chunk)
        self.chunk_steps = 0
        self.slice_s = float(slice_ms) / 1e3
        self.sliced = self.slice_s > 0 and self.prefill_chunk > 1
        self.sessions = sessions
        self.clock = clock
        self.bc = model.make_cache(max_rows=max_rows, n_pages=n_pages, max_pages_per_row=max_pages_per_row)
        # sliced prefill: the request being prefilled lives on a one-row cache of its own until its prompt is through
        self.pc = model.make_cache(max_rows=1, n_pages=max_pages_per_row, max_pages_per_row=max_pages_per_row) if self.sliced else None
        self.prefilling: deque = deque()
        self._gen, self._gen_n = None, 0
        self.spec, self.spec_T, self.bspec_max, self.bspec_rows = bool(spec), int(spec_T), int(bspec_max), int(bspec_rows)
        self.drafter_factory = drafter_factory
        self.stats = {"slices": 0, "slice_layers_max": 0, "resumed_tokens": 0, "snapshots": 0, "stall_s_max": 0.0,
                      "spec_steps": 0, "spec_rows": 0, "spec_drafted": 0, "spec_accepted": 0, "decode_steps": 0}
        self._last_decode = None
        self.n_pages, self.max_pages_per_row = n_pages, max_pages_per_row
        self.waiting: deque = deque()
        self.running: dict = {}
        self.finished: dict = {}
        self.reserved = 0          # pages promised to the running requests (their worst case)
        self._next = 0

    def warm_graphs(self):
        """Captures the decode step's CUDA graph for every batch size 1 .. max_rows before any request arrives (a graph
        is captured the first time its batch size is stepped, about a third of a second for the 72-layer model, which
        would otherwise fall between two decode steps of the running rows). Placeholder rows join one by one, take one
        step each time, and leave; their pages go back to the pool. The reference pays this cost per step instead (it
        rebuilds a lazy graph every step and pipelines the host work, batch.py:518-554)."""
        assert not self.running and not self.prefilling, "only on an idle engine"
        keys = [("warm", i) for i in range(self.bc.S)]
        for i, k in enumerate(keys):
            self.bc.apply(join=[k])
            BT.forward(self.model, self.bc, [0] * (i + 1))
        self.bc.apply(leave=keys)

    def _pages(self, r: Request) -> int:
        return (len(r.prompt) + r.max_new + PAGE - 1) // PAGE

    def submit(self, prompt, max_new, session=None) -> int:
        assert len(prompt) >= 1 and max_new >= 1
        r = Request(self._next, [int(t) for t in prompt], int(max_new), session=session)
        assert self._pages(r) <= self.max_pages_per_row, "request longer than a row's page table"
        self._next += 1
        self.waiting.append(r)
        return r.key

    def _admit(self):
        join = []
        while self.waiting and len(self.running) + len(self.prefilling) + len(join) < self.bc.S:
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
            self._snapshot_reply(r)
        if self.sliced:
            return self._sliced_step(leave)
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

    # ------------------------------------------------------------------ sliced prefill on a cache of its own
    def _sync(self):
        torch.cuda.current_stream().synchronize()

    def _snapshot_reply(self, r):
        """End of a reply: the row holds prompt + reply minus the last token (scheduler.py:504-560)."""
        if self.sessions is None or not self.sessions.enabled or r.key not in self.bc.keys:
            return
        toks = (r.prompt + r.out)[:-1]
        if not self.sessions.has(toks):
            self.sessions.add(r.session, "reply", toks, self.bc.capture_row(r.key))
            self.stats["snapshots"] += 1

    def _start_prefill(self, r):
        """Put request r on the prefill cache: fresh, or from the longest snapshot that is a prefix of its prompt."""
        snap = self.sessions.find(r.prompt, r.session) if self.sessions is not None else None
        state = None
        if snap is not None:
            state = snap.state
            r.fed = r.resumed = snap.pos
            self.stats["resumed_tokens"] += snap.pos
        self.pc.apply(join=[(r.key, state)])
        if self.sessions is not None:
            r.points = self.sessions.points(r.fed, len(r.prompt))
        return snap

    def _finish_prefill(self, r, first, logits):
        """The prompt is through: snapshot, then move the row into the decode batch."""
        st = self.pc.capture_row(r.key, logits=logits)
        if self.sessions is not None and self.sessions.enabled and not self.sessions.has(r.prompt):
            self.sessions.add(r.session, "prompt", r.prompt, st)
            self.stats["snapshots"] += 1
        self.pc.apply(leave=[r.key])
        self.bc.apply(join=[(r.key, st)])
        r.out.append(first)
        self.running[r.key] = r

    def _prefill_work(self, produced):
        """Prefill layers of the oldest admitted request: without a limit while nothing decodes (one chunk per tick),
        else until the slice is spent, stopping at a layer boundary (scheduler.py:241-263)."""
        decoding = bool(self.running)
        t_end = self.clock() + self.slice_s if decoding else None
        T = self.prefill_chunk
        layers = 0
        while self.prefilling:
            r = self.prefilling[0]
            if self._gen is None:
                if r.key not in self.pc.keys:
                    snap = self._start_prefill(r)
                    if r.fed >= len(r.prompt):       # the snapshot held the whole prompt and its last logits
                        st = self.pc.capture_row(r.key)
                        first = int(torch.argmax(snap.state.logits[: self.model.args.vocab_valid].float()))
                        self.pc.apply(leave=[r.key])
                        self.bc.apply(join=[(r.key, st)])
                        r.out.append(first)
                        self.running[r.key] = r
                        self.prefilling.popleft()
                        produced.append((r.key, first))
                        continue
                stop = min(len(r.prompt), r.fed + T, r.points[0] if r.points else len(r.prompt))
                chunk = r.prompt[r.fed:stop]
                self._gen_n = len(chunk)
                self._gen = CH.forward_chunk_iter(self.model, self.pc, [chunk], write=True, logits_at=[len(chunk) - 1])
            try:
                while True:
                    next(self._gen)
                    layers += 1
                    if t_end is not None:
                        self._sync()
                        if self.clock() >= t_end:
                            self.stats["slices"] += 1
                            self.stats["slice_layers_max"] = max(self.stats["slice_layers_max"], layers)
                            return
            except StopIteration as e:
                logits, greedy, _ = e.value
            self._gen = None
            r.fed += self._gen_n
            self.chunk_steps += 1
            if r.points and r.fed == r.points[0]:      # an interval snapshot inside a long prompt
                r.points.pop(0)
                if not self.sessions.has(r.prompt[: r.fed]):
                    self.sessions.add(r.session, "interval", r.prompt[: r.fed], self.pc.capture_row(r.key))
                    self.stats["snapshots"] += 1
            if r.fed >= len(r.prompt):
                first = int(greedy[0][0])
                self._finish_prefill(r, first, logits[0, 0] if logits is not None else None)
                self.prefilling.popleft()
                produced.append((r.key, first))
            if t_end is None:
                return                                  # nothing decodes: one chunk per tick
            self._sync()
            if self.clock() >= t_end:
                self.stats["slices"] += 1
                self.stats["slice_layers_max"] = max(self.stats["slice_layers_max"], layers)
                return

    def _sliced_step(self, leave):
        for r in self._admit():
            self.prefilling.append(r)
        if leave:
            self.bc.apply(leave=leave)
        produced = []
        self._prefill_work(produced)
        if self.bc.B:
            rows = [self.running[k] for k in self.bc.keys]
            live = [r for r in rows if not r.done]
            if live and self.spec and len(rows) <= self.bspec_max and self._spec_step(rows, produced):
                pass
            elif live:
                toks = [r.out[-1] for r in rows]
                self.stats["decode_steps"] += 1
                BT.forward(self.model, self.bc, toks)
                greedy = self.bc.greedy[: self.bc.B].tolist()
                now = self.clock()
                if self._last_decode is not None:
                    self.stats["stall_s_max"] = max(self.stats["stall_s_max"], now - self._last_decode)
                self._last_decode = now
                for r, g in zip(rows, greedy):
                    if not r.done:
                        r.out.append(int(g))
                        produced.append((r.key, int(g)))
        else:
            self._last_decode = None
        return produced

    def _spec_step(self, rows, produced) -> bool:
        """One batched speculative step of the decoding rows (scheduler.py:432-503). Returns False (nothing done) when
        no row has anything to propose."""
        T = max(2, min(self.spec_T, self.bspec_rows // len(rows)))
        drafts, any_draft = [], False
        for r in rows:
            if r.drafter is None or r.drafter_len != len(r.out):      # (re)entering: a fresh history
                r.drafter = self.drafter_factory()
                r.drafter.reset(r.prompt + r.out)
                r.drafter_len = len(r.out)
            d = [] if r.done else [int(t) for t in r.drafter.propose(T - 1)][: T - 1]
            any_draft = any_draft or bool(d)
            drafts.append(d)
        if not any_draft:
            for r in rows:
                r.drafter_len = -1        # (the plain step below appends a token the drafter has not seen)
            return False
        # a row with fewer drafts repeats its bonus token in the unused places: they are verified and (almost surely) rejected
        ids = [[r.out[-1]] + d + [r.out[-1]] * (T - 1 - len(d)) for r, d in zip(rows, drafts)]
        _, _, rec = SP.verify_forward(self.model, self.bc, ids)
        tok = rec.greedy.tolist()
        ns = []
        emitted = []
        for b, r in enumerate(rows):
            n = 1
            while n < T and n - 1 < len(drafts[b]) and ids[b][n] == tok[b][n - 1]:
                n += 1
            em = ids[b][1:n] + [tok[b][n - 1]]          # accepted drafts + the model's own next token
            em = em[: max(0, r.max_new - len(r.out))]
            emitted.append(em)
            ns.append(max(1, len(em)))
        SP.commit(self.bc, rec, ns)
        self.stats["spec_steps"] += 1
        self.stats["spec_rows"] += len(rows)
        for b, r in enumerate(rows):
            self.stats["spec_drafted"] += len(drafts[b])
            self.stats["spec_accepted"] += max(0, len(emitted[b]) - 1)
            r.drafter.record(emitted[b])
            for t in emitted[b]:
                r.out.append(int(t))
                produced.append((r.key, int(t)))
            r.drafter_len = len(r.out)
        now = self.clock()
        if self._last_decode is not None:
            self.stats["stall_s_max"] = max(self.stats["stall_s_max"], now - self._last_decode)
        self._last_decode = now
        return True

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
        while (self.waiting or self.running or self.prefilling) and n < max_steps:
            self.step()
            n += 1
            if all(r.done for r in self.running.values()) and not self.waiting and not self.prefilling:
                for k in list(self.running):
                    r = self.running.pop(k)
                    self.reserved -= self._pages(r)
                    self.finished[k] = r
                    self._snapshot_reply(r)
                if self.bc.B:
                    self.bc.apply(leave=list(self.bc.keys))
        return {k: r.out for k, r in self.finished.items()}
