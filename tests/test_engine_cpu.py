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
