"""Host logic of the continuous-batching engine (volundr_mlx_b200.engine) without a GPU: a fake cache and a fake step
whose "greedy token" is a function of the row's own history, so that any mix-up of rows, prompts or positions under
joins, leaves and queueing changes a request's output."""
import torch

from volundr_mlx_b200 import engine as E


class FakeCache:
    def __init__(self, S):
        self.S, self.keys, self.hist = S, [], {}
        self.greedy = torch.zeros(S, dtype=torch.int32)

    @property
    def _pos(self):
        return [len(self.hist[k]) for k in self.keys]

    @property
    def B(self):
        return len(self.keys)

    def apply(self, leave=(), join=()):
        for k in leave:            # swap-remove, as the real cache does
            b = self.keys.index(k)
            self.keys[b] = self.keys[-1]
            self.keys.pop()
            del self.hist[k]
        for k in join:
            assert self.B < self.S
            self.keys.append(k)
            self.hist[k] = []


class FakeModel:
    def make_cache(self, max_rows, n_pages, max_pages_per_row):
        return FakeCache(max_rows)


def fake_next(hist):
    return (sum((i + 1) * t for i, t in enumerate(hist)) * 31 + len(hist)) % 997


def fake_forward(model, bc, toks):
    assert len(toks) == bc.B
    for b, k in enumerate(bc.keys):
        bc.hist[k].append(int(toks[b]))
        bc.greedy[b] = fake_next(bc.hist[k])


def solo(prompt, max_new):
    hist, out = [], []
    for t in prompt:
        hist.append(t)
    out.append(fake_next(hist))
    while len(out) < max_new:
        hist.append(out[-1])
        out.append(fake_next(hist))
    return out


def test_engine_rows_are_independent_under_queueing(monkeypatch):
    monkeypatch.setattr(E.BT, "forward", fake_forward)
    eng = E.BatchEngine(FakeModel(), max_rows=3, n_pages=6, max_pages_per_row=2)
    reqs = [([5, 6, 7], 4), ([1], 9), ([9, 8, 7, 6, 5, 4, 3], 2), ([2, 2], 1), ([3, 1, 4, 1, 5], 6), (list(range(1, 70)), 3)]
    keys = [eng.submit(p, n) for p, n in reqs]
    peak = 0
    steps = 0
    while eng.waiting or eng.running:
        eng.step()
        steps += 1
        peak = max(peak, eng.bc.B)
        assert eng.bc.B <= 3 and eng.reserved <= 6
        assert steps < 500
        if all(r.done for r in eng.running.values()) and not eng.waiting:
            break
    out = eng.run()
    assert peak == 3
    for k, (p, n) in zip(keys, reqs):
        assert out[k] == solo(p, n), k
    assert eng.reserved == 0 and eng.bc.B == 0


def test_warm_graphs_leaves_the_engine_empty(monkeypatch):
    """Pre-capturing steps every batch size once with placeholder rows and gives everything back: requests served
    afterwards get the same tokens as without it."""
    monkeypatch.setattr(E.BT, "forward", fake_forward)
    sizes = []
    real_forward = E.BT.forward
    monkeypatch.setattr(E.BT, "forward", lambda m, bc, toks: (sizes.append(len(toks)), real_forward(m, bc, toks))[1])
    eng = E.BatchEngine(FakeModel(), max_rows=3, n_pages=64, max_pages_per_row=8)
    eng.warm_graphs()
    assert sizes == [1, 2, 3] and eng.bc.B == 0 and not eng.bc.hist
    prompts = [[5, 6, 7], [9], [1, 2]]
    for p_ in prompts:
        eng.submit(p_, 4)
    out = eng.run()
    assert [out[i] for i in range(3)] == [solo(p_, 4) for p_ in prompts]


def test_engine_waits_for_pages(monkeypatch):
    monkeypatch.setattr(E.BT, "forward", fake_forward)
    eng = E.BatchEngine(FakeModel(), max_rows=4, n_pages=2, max_pages_per_row=2)
    a = eng.submit(list(range(1, 100)), 20)    # 2 pages: fills the pool
    b = eng.submit([1, 2], 2)                  # has to wait although rows are free
    eng.step()
    assert list(eng.running) == [a] and len(eng.waiting) == 1
    out = eng.run()
    assert out[a] == solo(list(range(1, 100)), 20) and out[b] == solo([1, 2], 2)


def fake_forward_chunk(model, bc, toks, write=False, logits_at=None):
    """The chunk interface on the fake cache: one list of tokens per row (ragged); greedy[b][0] follows the row's
    history plus its tokens up to index logits_at[b]; the engine commits every chunk as it is (write=True)."""
    assert write and len(toks) == bc.B and len(logits_at) == bc.B and all(len(t) >= 1 for t in toks)
    greedy = torch.zeros((bc.B, 1), dtype=torch.int32)
    for b, k in enumerate(bc.keys):
        assert 0 <= logits_at[b] < len(toks[b])
        greedy[b, 0] = fake_next(bc.hist[k] + [int(x) for x in toks[b][: logits_at[b] + 1]])
        bc.hist[k] += [int(x) for x in toks[b]]
    return None, greedy, None


def test_engine_ragged_prefill_chunks(monkeypatch):
    """Prompts fed in chunks of up to 4 tokens per row while other rows decode: every request still gets its solo
    output, prompt tokens go through chunk steps, and a chunk never outgrows a row's page table or the pool."""
    monkeypatch.setattr(E.BT, "forward", fake_forward)
    monkeypatch.setattr(E.CH, "forward_chunk", fake_forward_chunk)
    eng = E.BatchEngine(FakeModel(), max_rows=3, n_pages=6, max_pages_per_row=2, prefill_chunk=4)
    reqs = [([5, 6, 7], 4), ([1], 9), ([9, 8, 7, 6, 5, 4, 3], 2), ([2, 2], 1), ([3, 1, 4, 1, 5], 6), (list(range(1, 70)), 3),
            (list(range(1, 126)), 3)]
    keys = [eng.submit(p, n) for p, n in reqs]
    steps = 0
    while eng.waiting or eng.running:
        eng.step()
        steps += 1
        assert all(p <= 2 * E.PAGE for p in eng.bc._pos)
        assert steps < 500
        if all(r.done for r in eng.running.values()) and not eng.waiting:
            break
    out = eng.run()
    for k, (p, n) in zip(keys, reqs):
        assert out[k] == solo(p, n), k
    assert eng.chunk_steps >= (69 + 125) // 4 // 3
    assert steps < sum(len(p) + n for p, n in reqs) // 3     # far fewer steps than one token per step would take


# ---------------------------------------------------------------------------------- sliced prefill, sessions (fakes)
class FakeState:
    def __init__(self, hist, logits=None):
        self.hist, self.logits, self.pos, self.nbytes = list(hist), logits, len(hist), 8 * len(hist) + 8


class SlicedFakeCache(FakeCache):
    """apply(join=[(key, state)]) / capture_row as the real cache offers them."""

    def apply(self, leave=(), join=()):
        plain = []
        for item in join:
            if isinstance(item, tuple):
                k, st = item
                assert self.B + len(plain) < self.S
                self.keys.append(k)
                self.hist[k] = list(st.hist) if st is not None else []
            else:
                plain.append(item)
        super().apply(leave=leave, join=plain)

    def capture_row(self, key, logits=None):
        return FakeState(self.hist[key], logits)


class SlicedFakeModel:
    class args:
        vocab_valid = 997

    def make_cache(self, max_rows, n_pages, max_pages_per_row):
        return SlicedFakeCache(max_rows)


LAYERS = 5


def fake_forward_chunk_iter(model, bc, toks, write=False, logits_at=None, capture=(), yield_layers=True):
    """A chunk pass of LAYERS layers that hands control back after every layer but the last; the cache only changes when
    the pass completes."""
    assert write and len(toks) == bc.B == 1 and logits_at == [len(toks[0]) - 1]
    for i in range(LAYERS - 1):
        yield ("layer", i)
    k = bc.keys[0]
    bc.hist[k] += [int(x) for x in toks[0]]
    g = fake_next(bc.hist[k])
    logits = torch.zeros(1, 1, 997)
    logits[0, 0, g] = 1.0
    return logits, torch.tensor([[g]], dtype=torch.int32), None


def _sliced_engine(monkeypatch, sessions=None, slice_layers=3, **kw):
    monkeypatch.setattr(E.BT, "forward", fake_forward)
    monkeypatch.setattr(E.CH, "forward_chunk_iter", fake_forward_chunk_iter)
    clock = {"t": 0.0, "log": []}
    eng = E.BatchEngine(SlicedFakeModel(), prefill_chunk=4, slice_ms=1000.0 * slice_layers, sessions=sessions,
                        clock=lambda: clock["t"], **kw)

    def sync():                     # every layer the engine waits for costs one unit of (fake) time
        clock["t"] += 1.0
        clock["log"].append("L")
    eng._sync = sync
    real_forward = E.BT.forward

    def logged_forward(model, bc, toks):
        clock["log"].append("D")
        return real_forward(model, bc, toks)
    monkeypatch.setattr(E.BT, "forward", logged_forward)
    return eng, clock


def test_sliced_prefill_interleaves_with_decode(monkeypatch):
    """While rows decode, no more than a slice's worth of prefill layers (+ the one that overruns it) runs between two
    decode steps, a chunk is resumed where it stopped, and every request still gets its solo output."""
    eng, clock = _sliced_engine(monkeypatch, slice_layers=3, max_rows=3, n_pages=8, max_pages_per_row=2)
    reqs = [([5, 6, 7], 30), (list(range(1, 60)), 4), ([9, 8, 7, 6, 5, 4, 3, 2, 1], 3), (list(range(3, 40)), 2)]
    keys = [eng.submit(p, n) for p, n in reqs]
    out = eng.run()
    for k, (p, n) in zip(keys, reqs):
        assert out[k] == solo(p, n), k
    log = "".join(clock["log"])
    assert "D" in log and "L" in log
    # between two decode steps: at most slice_layers layers are waited for (the slice ends at the first layer boundary
    # at or past the deadline)
    runs = [len(x) for x in log.strip("L").split("D") if x]
    assert runs and max(runs) <= 3, runs
    assert eng.stats["slices"] > 0 and eng.stats["slice_layers_max"] <= 3
    assert eng.reserved == 0 and eng.bc.B == 0 and eng.pc.B == 0


def test_sessions_resume_from_longest_prefix(monkeypatch):
    from volundr_mlx_b200.session import SessionCache

    sc = SessionCache(budget_gb=1.0, interval=16, min_gap=4)
    eng, _ = _sliced_engine(monkeypatch, sessions=sc, max_rows=2, n_pages=8, max_pages_per_row=4)
    first = list(range(1, 50))
    k1 = eng.submit(first, 5, session="s")
    out = eng.run()
    assert out[k1] == solo(first, 5)
    kinds = sorted(s.kind for s in sc.snaps)
    assert kinds == ["interval", "interval", "prompt", "reply"], kinds          # positions 16, 32; 49; 49 + 4
    # a follow-up turn: the first prompt, the reply, and new tokens: only the new tokens are prefilled
    reply = out[k1]
    follow = first + reply + [7, 7, 7]
    fed_before = eng.chunk_steps
    k2 = eng.submit(follow, 3, session="s")
    out = eng.run()
    assert out[k2] == solo(follow, 3)
    assert eng.finished[k2].resumed == len(first) + len(reply) - 1              # the end-of-reply snapshot
    assert eng.chunk_steps - fed_before == 1                                    # 4 tokens left: one chunk
    # the very same prompt again: nothing is prefilled, the first token comes from the snapshot's logits
    fed_before = eng.chunk_steps
    k3 = eng.submit(first, 2, session="other")
    out = eng.run()
    assert out[k3] == solo(first, 2) and eng.chunk_steps == fed_before
    assert eng.stats["resumed_tokens"] >= len(first)


def test_session_cache_budget_and_lookup():
    import numpy as np
    from volundr_mlx_b200.session import SessionCache

    sc = SessionCache(budget_gb=1e-6, interval=8, min_gap=2)     # 1000 bytes
    mk = lambda n: FakeState(list(range(n)))
    a = sc.add("a", "prompt", list(range(10)), mk(10))          # 88 + 40 bytes
    b = sc.add("b", "prompt", list(range(20)), mk(20))
    assert a is not None and b is not None
    assert sc.find(list(range(30)), "a") is b                    # the longest prefix wins over the own session
    assert sc.find(list(range(10)), "a") is None                 # nothing left to feed and no logits kept
    assert sc.find(list(range(15)), "zz") is a
    assert sc.find([1, 2, 3], "a") is None
    assert sc.points(0, 30) == [8, 16, 24] and sc.points(10, 30) == [16, 24] and sc.points(0, 9) == []
    for n in range(21, 40):                                      # overflow the budget: least recently used go first
        sc.add("c", "prompt", list(range(n)), mk(n))
    assert sc.nbytes <= sc.budget and sc.evicted > 0
    assert sc.find(list(range(100)), None).pos == 39
    assert sc.add("d", "prompt", list(range(1000)), mk(1000)) is None   # larger than the whole budget


# ---------------------------------------------------------------------------------- batched speculative steps (fakes)
class FakeRec:
    pass


def fake_verify_forward(model, bc, ids, capture=()):
    rec = FakeRec()
    rec.ids = [list(map(int, row)) for row in ids]
    T = len(rec.ids[0])
    g = torch.zeros((bc.B, T), dtype=torch.int32)
    for b, k in enumerate(bc.keys):
        for t in range(T):
            g[b, t] = fake_next(bc.hist[k] + rec.ids[b][: t + 1])
    rec.greedy = g
    return None, None, rec


def fake_commit(bc, rec, ns):
    for b, k in enumerate(bc.keys):
        assert 1 <= ns[b] <= len(rec.ids[b])
        bc.hist[k] += rec.ids[b][: ns[b]]


class OracleDrafter:
    """Drafts the true continuation for the first `good` places of a proposal, garbage after (good = 99: perfect)."""
    good = 99

    def reset(self, ids):
        self.hist = list(ids)

    def propose(self, k):
        h, out = list(self.hist), []
        for i in range(k):
            t = fake_next(h)
            out.append(t if i < self.good else (t + 1) % 997)
            h.append(t)
        return out

    def record(self, emitted):
        self.hist.extend(emitted)


def test_speculative_steps_keep_the_greedy_sequence(monkeypatch):
    from volundr_mlx_b200.lookup import Lookup

    for good, factory in ((99, OracleDrafter), (2, OracleDrafter), (0, OracleDrafter), (None, Lookup)):
        if good is not None:
            OracleDrafter.good = good
        eng, _ = _sliced_engine(monkeypatch, max_rows=3, n_pages=12, max_pages_per_row=4)
        monkeypatch.setattr(E.SP, "verify_forward", fake_verify_forward)
        monkeypatch.setattr(E.SP, "commit", fake_commit)
        eng.spec, eng.spec_T, eng.bspec_max, eng.bspec_rows, eng.drafter_factory = True, 8, 4, 16, factory
        reqs = [([5, 6, 7], 30), (list(range(1, 60)), 17), ([9, 8, 7, 6, 5, 4, 3, 2, 1], 23), ([4, 4, 4, 4, 4, 4, 4], 9)]
        keys = [eng.submit(p, n) for p, n in reqs]
        out = eng.run()
        for k, (p, n) in zip(keys, reqs):
            assert out[k] == solo(p, n), (good, k)
        if good == 99:       # every draft accepted: far fewer steps than tokens
            # (all but the drafts that ran past a request's last token)
            assert eng.stats["spec_drafted"] - 7 * len(reqs) <= eng.stats["spec_accepted"] <= eng.stats["spec_drafted"] > 0
            assert eng.stats["spec_steps"] + eng.stats["decode_steps"] < sum(n for _, n in reqs) // 2
        elif good == 2:
            assert 0 < eng.stats["spec_accepted"] < eng.stats["spec_drafted"]
        elif good == 0:
            assert eng.stats["spec_accepted"] == 0 and eng.stats["spec_steps"] > 0


def test_lookup_proposes_what_followed_the_longest_match():
    from volundr_mlx_b200.lookup import Lookup, bucket_of

    lk = Lookup(min_gain=0.0)
    seq = [1, 2, 3, 4, 5, 9, 9, 2, 3, 4, 7, 8, 1, 2, 3, 4]
    lk.reset(seq)
    cont, m = lk.find()
    assert m == 4 and cont[:2] == [5, 9]            # "1 2 3 4" at the start beats "2 3 4" in the middle
    assert lk.propose(3) == [5, 9, 9]
    lk.record([5, 9, 1])                            # two of three accepted, then the model's own token
    assert lk.hist[-3:] == [5, 9, 1] and lk.accepted == 2
    assert [bucket_of(m) for m in (1, 2, 3, 5, 6, 9, 10, 64)] == [0, 0, 1, 2, 3, 3, 4, 5]
    lk.reset([1, 2])
    assert lk.propose() == []                       # too short to match anything
    strict = Lookup(min_gain=10.0)
    strict.reset(seq)
    assert strict.propose() == []                   # a match, but not expected to pay
