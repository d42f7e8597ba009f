"""Continuous batching on the GPU (volundr_mlx_b200.engine over batch.forward): requests with different prompt and
output lengths share three rows, queue, join and leave; every request must generate exactly the tokens it generates
alone on a one-row cache (the property the reference pins for its batch path, test_batch.py:49-116: each row equals
its own B = 1 run), here bit for bit because every kernel's result for a row is independent of the other rows."""
import numpy as np
import pytest
import torch

from volundr_mlx_b200 import synth

pytestmark = pytest.mark.gpu


def test_engine_equals_solo_runs():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from volundr_mlx_b200 import batch as BT, ops
    from volundr_mlx_b200.engine import BatchEngine
    from volundr_mlx_b200.volundr import Model

    cuda = torch.device("cuda", 0)
    args = synth.small_args(bcsa_far="tokens", bcsa_score="pooled_key", bcsa_window=128, bcsa_compress=64, bcsa_topk=2)
    params = synth.make_params(args, seed=21)
    model = Model(args, params, cuda)
    rng = np.random.default_rng(21)
    reqs = [(rng.integers(0, args.vocab_valid, size=n).tolist(), m)
            for n, m in [(70, 12), (3, 40), (130, 5), (1, 8), (25, 25), (64, 64)]]
    eng = BatchEngine(model, max_rows=3, n_pages=24, max_pages_per_row=4)
    keys = [eng.submit(p, m) for p, m in reqs]
    out = eng.run()
    ops.check_status()
    for k, (prompt, m) in zip(keys, reqs):
        one = model.make_cache(max_rows=1, n_pages=8, max_pages_per_row=4)
        one.apply(join=["x"])
        for t in prompt:
            BT.forward(model, one, [t])
        want = [int(one.greedy[0])]
        while len(want) < m:
            BT.forward(model, one, [want[-1]])
            want.append(int(one.greedy[0]))
        assert out[k] == want, k
    ops.check_status()


def test_engine_prefill_chunks():
    """The same requests with prompts fed in ragged chunks of up to 32 tokens per row (engine.BatchEngine with
    prefill_chunk: one pass over the weights per chunk, decoding rows ride along with one token) against the solo
    stepwise runs. The chunk path's GEMMs round differently from the decode step's, so the tokens must agree up to the
    first near-tie: where a request's tokens first differ, the token the engine chose must lie within 0.05 of the
    maximum of the stepwise logits at that position (the bf16 bar 2e-2 on logits of magnitude about one, twice)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from volundr_mlx_b200 import batch as BT, ops
    from volundr_mlx_b200.engine import BatchEngine
    from volundr_mlx_b200.volundr import Model

    cuda = torch.device("cuda", 0)
    args = synth.small_args(bcsa_far="tokens", bcsa_score="pooled_key", bcsa_window=128, bcsa_compress=64, bcsa_topk=2)
    params = synth.make_params(args, seed=22)
    model = Model(args, params, cuda)
    rng = np.random.default_rng(22)
    reqs = [(rng.integers(0, args.vocab_valid, size=n).tolist(), m)
            for n, m in [(70, 12), (3, 20), (130, 5), (1, 8), (33, 9), (64, 30)]]
    eng = BatchEngine(model, max_rows=3, n_pages=24, max_pages_per_row=4, prefill_chunk=32)
    keys = [eng.submit(p, m) for p, m in reqs]
    out = eng.run()
    ops.check_status()
    assert eng.chunk_steps >= 6        # (70 + 130 + 33 + 64 prompt tokens cannot go through fewer chunks of 32)
    same = 0
    for k, (prompt, m) in zip(keys, reqs):
        assert len(out[k]) == m
        one = model.make_cache(max_rows=1, n_pages=8, max_pages_per_row=4)
        one.apply(join=["x"])
        for t in prompt:
            lg, _ = BT.forward(model, one, [t])
        for j in range(m):
            lg = lg[0].float()
            want = int(one.greedy[0])
            if out[k][j] != want:
                assert float(lg.max() - lg[out[k][j]]) < 0.05, (k, j, float(lg.max() - lg[out[k][j]]))
                break
            if j + 1 < m:
                lg, _ = BT.forward(model, one, [want])
        else:
            same += 1
    assert same >= len(reqs) // 2, same
    ops.check_status()


def _solo_check(model, BT, prompt, got, m):
    """got == the stepwise solo tokens up to the first near-tie (see test_engine_prefill_chunks); returns True when all
    m tokens agree."""
    one = model.make_cache(max_rows=1, n_pages=8, max_pages_per_row=6)
    one.apply(join=["x"])
    for t in prompt:
        lg, _ = BT.forward(model, one, [t])
    for j in range(m):
        lg = lg[0].float()
        want = int(one.greedy[0])
        if got[j] != want:
            assert float(lg.max() - lg[got[j]]) < 0.05, (j, float(lg.max() - lg[got[j]]))
            return False
        if j + 1 < m:
            lg, _ = BT.forward(model, one, [want])
    return True


def test_engine_sliced_prefill_and_sessions():
    """Prompts prefilled on a cache of their own in chunks that stop at layer boundaries when the time slice is spent
    (scheduler.py:241-263), then joined into the decode batch as a State; with a session cache a follow-up turn resumes
    from the end-of-reply snapshot and prefills only its new tokens (scheduler.py:134-190, session.py:240-330)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from volundr_mlx_b200 import batch as BT, ops
    from volundr_mlx_b200.engine import BatchEngine
    from volundr_mlx_b200.session import SessionCache
    from volundr_mlx_b200.volundr import Model

    cuda = torch.device("cuda", 0)
    for mode_kw in (dict(bcsa_far="tokens", bcsa_score="pooled_key", bcsa_window=128, bcsa_compress=64, bcsa_topk=2), {}):
        args = synth.small_args(**mode_kw)
        params = synth.make_params(args, seed=23)
        model = Model(args, params, cuda)
        rng = np.random.default_rng(23)
        reqs = [(rng.integers(0, args.vocab_valid, size=n).tolist(), m)
                for n, m in [(70, 12), (3, 20), (200, 5), (1, 8), (33, 9), (64, 30)]]
        sc = SessionCache(budget_gb=0.5, interval=64, min_gap=8)
        # (a slice of 50 microseconds: every chunk is cut after its first layer or two while something decodes)
        eng = BatchEngine(model, max_rows=3, n_pages=32, max_pages_per_row=6, prefill_chunk=48, slice_ms=0.05, sessions=sc)
        keys = [eng.submit(p, m, session=f"s{i}") for i, (p, m) in enumerate(reqs)]
        out = eng.run()
        ops.check_status()
        assert eng.stats["slices"] > 0, eng.stats
        same = sum(_solo_check(model, BT, p, out[k], m) for k, (p, m) in zip(keys, reqs))
        assert same >= len(reqs) // 2, same
        assert {s.kind for s in sc.snaps} == {"prompt", "reply", "interval"}
        # follow-up turn of request 2: prompt + reply + new tokens; only the new tokens are prefilled
        p2, m2 = reqs[2]
        follow = p2 + out[keys[2]] + rng.integers(0, args.vocab_valid, size=5).tolist()
        chunks_before = eng.chunk_steps
        k = eng.submit(follow, 10, session="s2")
        out2 = eng.run()
        ops.check_status()
        assert eng.finished[k].resumed == len(p2) + m2 - 1
        assert eng.chunk_steps - chunks_before == 1
        _solo_check(model, BT, follow, out2[k], 10)
        assert eng.bc.B == 0 and eng.pc.B == 0 and eng.reserved == 0
        free = int(eng.bc.free_top.item())
        assert free == eng.bc.n_pages, "every page went back to the pool"


def test_engine_batched_speculative_steps():
    """Batched speculative steps (scheduler.py:432-503 over batch_spec.verify_forward / commit): rows draft, one verify
    pass checks all rows' drafts, each row keeps its accepted run. With a drafter that replays the request's true greedy
    continuation every draft must be accepted (up to near-ties between the verify pass and the decode step); with
    prompt lookup on repetitive prompts whatever is accepted, the emitted tokens stay the greedy sequence."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from volundr_mlx_b200 import batch as BT, ops
    from volundr_mlx_b200.engine import BatchEngine
    from volundr_mlx_b200.lookup import Lookup
    from volundr_mlx_b200.volundr import Model

    cuda = torch.device("cuda", 0)
    args = synth.small_args()
    params = synth.make_params(args, seed=24)
    model = Model(args, params, cuda)
    rng = np.random.default_rng(24)
    pat = rng.integers(0, args.vocab_valid, size=7).tolist()
    reqs = [(pat * 6, 24), (rng.integers(0, args.vocab_valid, size=40).tolist(), 30), (pat[::-1] * 9, 17)]
    # the greedy continuations, from solo stepwise runs
    truth = {}
    for i, (prompt, m) in enumerate(reqs):
        one = model.make_cache(max_rows=1, n_pages=8, max_pages_per_row=6)
        one.apply(join=["x"])
        for t in prompt:
            BT.forward(model, one, [t])
        seq = [int(one.greedy[0])]
        while len(seq) < m + 8:
            BT.forward(model, one, [seq[-1]])
            seq.append(int(one.greedy[0]))
        truth[tuple(prompt)] = seq

    class Replay:
        def reset(self, ids):
            self.ids = list(ids)

        def propose(self, k):
            for prompt, seq in truth.items():
                n = len(prompt)
                if tuple(self.ids[:n]) == prompt:
                    done = len(self.ids) - n
                    return seq[done: done + k] if self.ids[n:] == seq[:done] else []
            return []

        def record(self, emitted):
            self.ids.extend(emitted)

    for factory in (Replay, Lookup):
        eng = BatchEngine(model, max_rows=3, n_pages=32, max_pages_per_row=6, prefill_chunk=48, slice_ms=50.0, spec=True,
                          spec_T=8, bspec_max=4, bspec_rows=16, drafter_factory=factory)
        keys = [eng.submit(p, m) for p, m in reqs]
        out = eng.run()
        ops.check_status()
        same = sum(_solo_check(model, BT, p, out[k], m) for k, (p, m) in zip(keys, reqs))
        assert same >= 2, same
        assert all(len(out[k]) == m for k, (p, m) in zip(keys, reqs))
        if factory is Replay:
            assert eng.stats["spec_steps"] > 0
            assert eng.stats["spec_accepted"] >= 0.6 * eng.stats["spec_drafted"], eng.stats
            assert eng.stats["spec_steps"] + eng.stats["decode_steps"] < sum(m for _, m in reqs) // 2
        assert eng.bc.B == 0 and int(eng.bc.free_top.item()) == eng.bc.n_pages
