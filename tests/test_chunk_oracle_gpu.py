"""The T-tokens-per-row path (volundr_mlx_b200.chunk behind batch_spec.verify_forward / commit, and as prefill chunks)
against the CPU oracle run token by token: the logits of every position, the drafter features, and what a commit leaves
in the cache (K / V by position, pooled blocks, pooled and open-block indexer keys, KDA state and conv window, Engram
ids), then the logits of the decode steps that follow, far enough for the blocks closed inside the chunk to enter the
far range. Reference checks behind this: tests/test_batch.py:180-219 (per-row verify commit == sequential append),
tests/test_volundr.py:301-317 (the bf16 bar). Bars: logits rtol 2e-2 / atol 2e-2; state as seeding.assert_state_close."""
import copy

import numpy as np
import pytest
import torch

from oracle.model import Oracle
from volundr_mlx_b200 import synth

import seeding

pytestmark = pytest.mark.gpu

MODES = {"reference": {}, "paged_tokens": dict(bcsa_far="tokens", bcsa_score="pooled_key", bcsa_window=128, bcsa_compress=64,
                                               bcsa_topk=2)}


def _close(got, want, what):
    np.testing.assert_allclose(got, want, rtol=2e-2, atol=2e-2, err_msg=str(what))


def _warm(model, bc, orc, rows, keys, toks, BT):
    for t in range(toks.shape[0]):
        BT.forward(model, bc, toks[t].tolist())
        for r, k in enumerate(keys):
            orc.step(rows[k], int(toks[t, r]))


def _continue(model, bc, orc, rows, keys, toks, BT, what):
    for t in range(toks.shape[0]):
        lg, _ = BT.forward(model, bc, toks[t].tolist())
        got = lg.float().cpu().numpy()
        for r, k in enumerate(keys):
            _close(got[r], orc.step(rows[k], int(toks[t, r])), (what, "continue", t, k))


@pytest.mark.parametrize("mode", list(MODES))
def test_verify_and_commit_against_oracle(cuda, mode):
    from volundr_mlx_b200 import batch as BT, batch_spec as SP, ops
    from volundr_mlx_b200.volundr import Model

    args = synth.small_args(**MODES[mode])
    params = synth.make_params(args, seed=41)
    model = Model(args, params, cuda)
    orc = Oracle(args, params, exact=False)
    rng = np.random.default_rng(41)
    keys = ["a", "b", "c"]
    B, T, warm, cont = 3, 8, 58, 30          # the window covers positions 58..65: blocks close inside it, a page opens at 64
    capture = (1, 4)
    warm_toks = rng.integers(0, args.vocab_valid, size=(warm, B))
    drafts = rng.integers(0, args.vocab_valid, size=(B, T))
    cont_toks = rng.integers(0, args.vocab_valid, size=(cont, B))
    accepted = [3, 8, 5]                     # 3 and 5: short of a block boundary of C = 4 (positions 61 and 63 are next)

    bc = model.make_cache(max_rows=4, n_pages=16, max_pages_per_row=4)
    bc.apply(join=keys)
    rows = {k: orc.new_row() for k in keys}
    _warm(model, bc, orc, rows, keys, warm_toks, BT)
    free_before = int(bc.free_top.item())

    logits, feats, rec = SP.verify_forward(model, bc, torch.from_numpy(drafts), capture=capture)
    ops.check_status()
    assert logits.shape == (B, T, model.vocab_shard) and feats.shape == (B, T, len(capture) * args.hidden_size)
    assert bc.host_pos() == [warm] * B, "a verify pass moves no position"
    got, gf = logits.float().cpu().numpy(), feats.float().cpu().numpy()
    greedy = rec.greedy.cpu().numpy()
    for r, k in enumerate(keys):
        probe = copy.deepcopy(rows[k])       # all T drafts through the oracle: what the verify pass must reproduce
        for t in range(T):
            want, wf = orc.step(probe, int(drafts[r, t]), capture=capture)
            _close(got[r, t], want, (mode, "verify", k, t))
            seeding._close(gf[r, t], wf, 2e-2, (mode, "features", k, t))   # (residual streams: a fraction of their scale)
            assert greedy[r, t] == int(np.argmax(got[r, t][: args.vocab_valid]))
    SP.commit(bc, rec, accepted)
    for r, k in enumerate(keys):             # the oracle keeps the same prefixes
        for t in range(accepted[r]):
            orc.step(rows[k], int(drafts[r, t]))
    assert bc.host_pos() == [warm + n for n in accepted]
    assert int(bc.free_top.item()) == free_before - sum(1 for n in accepted if warm + n > 64)
    for k in keys:
        seeding.assert_state_close(bc, k, rows[k], args, what=(mode, "after commit", k))
    _continue(model, bc, orc, rows, keys, cont_toks, BT, mode)
    ops.check_status()
    for k in keys:
        seeding.assert_state_close(bc, k, rows[k], args, what=(mode, "after continuing", k))


@pytest.mark.parametrize("mode", list(MODES))
def test_prefill_chunks_against_oracle(cuda, mode):
    """A 200-token prompt in chunks of 96, 48 and 56 tokens (the first one runs the tcgen05 tile GEMM, the others the
    streaming kernel's row passes; every chunk spans many blocks of C = 4 positions in the reference form)."""
    from volundr_mlx_b200 import batch as BT, chunk as CH, ops
    from volundr_mlx_b200.volundr import Model

    args = synth.small_args(**MODES[mode])
    params = synth.make_params(args, seed=42)
    model = Model(args, params, cuda)
    orc = Oracle(args, params, exact=False)
    rng = np.random.default_rng(42)
    prompt = rng.integers(0, args.vocab_valid, size=200).tolist()
    tail = rng.integers(0, args.vocab_valid, size=(30, 1))
    bc = model.make_cache(max_rows=1, n_pages=8, max_pages_per_row=6)
    bc.apply(join=["x"])
    row = orc.new_row()
    c0 = 0
    for n in (96, 48, 56):
        lg, greedy, _ = CH.forward_chunk(model, bc, [prompt[c0:c0 + n]], write=True)
        got = lg.float().cpu().numpy()[0]
        for t in range(n):
            _close(got[t], orc.step(row, prompt[c0 + t]), (mode, "chunk at", c0, t))
        c0 += n
        ops.check_status()
        seeding.assert_state_close(bc, "x", row, args, what=(mode, "after chunk ending at", c0))
    assert bc.host_pos() == [200]
    _continue(model, bc, orc, {"x": row}, ["x"], tail, BT, mode)
    ops.check_status()


def test_ragged_chunk_against_oracle(cuda):
    """Rows that bring 1, 70 and 9 tokens (a decoding row beside two prompt rows), once committed as they are and once
    as a verify pass that keeps 1, 33 and 0 of them."""
    from volundr_mlx_b200 import batch as BT, chunk as CH, ops
    from volundr_mlx_b200.volundr import Model

    args = synth.small_args()
    params = synth.make_params(args, seed=43)
    model = Model(args, params, cuda)
    orc = Oracle(args, params, exact=False)
    rng = np.random.default_rng(43)
    keys = ["a", "b", "c"]
    warm, lens, cont = 21, [1, 70, 9], 24
    warm_toks = rng.integers(0, args.vocab_valid, size=(warm, 3))
    toks = [rng.integers(0, args.vocab_valid, size=n).tolist() for n in lens]
    cont_toks = rng.integers(0, args.vocab_valid, size=(cont, 3))
    for kept in (None, [1, 33, 0]):
        bc = model.make_cache(max_rows=4, n_pages=16, max_pages_per_row=4)
        bc.apply(join=keys)
        rows = {k: orc.new_row() for k in keys}
        _warm(model, bc, orc, rows, keys, warm_toks, BT)
        if kept is None:
            logits, _, _ = CH.forward_chunk(model, bc, toks, write=True)
            kept_n = lens
        else:
            logits, _, h = CH.forward_chunk(model, bc, toks, write=False)
            CH.commit_chunk(model, bc, h, kept)
            kept_n = kept
        got = logits.float().cpu().numpy()
        for r, k in enumerate(keys):
            probe = copy.deepcopy(rows[k])
            want = None
            for t in range(lens[r]):
                want = orc.step(probe, toks[r][t])
            _close(got[r, 0], want, ("ragged", kept, k))       # the logits after the row's last token
            for t in range(kept_n[r]):
                orc.step(rows[k], toks[r][t])
        assert bc.host_pos() == [warm + n for n in kept_n]
        ops.check_status()
        for k in keys:
            seeding.assert_state_close(bc, k, rows[k], args, what=("ragged", kept, k))
        _continue(model, bc, orc, rows, keys, cont_toks, BT, ("ragged", kept))
    ops.check_status()


def test_join_of_a_captured_row_continues_bit_identically(cuda):
    """capture_row -> leave -> join (the scheduler's way of moving a request between caches, scheduler.py:328, :534;
    the reference checks test_session.py:58-81 and test_batch.py:104-116): the row lands in other pages and another
    slot, and its logits over the next steps equal, bit for bit, those of the row that never left."""
    from volundr_mlx_b200 import batch as BT, ops
    from volundr_mlx_b200.volundr import Model

    for mode in MODES:
        args = synth.small_args(**MODES[mode])
        params = synth.make_params(args, seed=44)
        model = Model(args, params, cuda)
        rng = np.random.default_rng(44)
        warm, cont = 150 if mode == "paged_tokens" else 70, 12
        warm_toks = rng.integers(0, args.vocab_valid, size=(warm, 3))
        cont_toks = rng.integers(0, args.vocab_valid, size=(cont, 3))
        stay = model.make_cache(max_rows=4, n_pages=32, max_pages_per_row=4)
        move = model.make_cache(max_rows=4, n_pages=32, max_pages_per_row=4, seed=1)
        for bc in (stay, move):
            bc.apply(join=["a", "b", "c"])
            for t in range(warm):
                BT.forward(model, bc, warm_toks[t].tolist())
        st = move.capture_row("b")
        assert st.pos == warm and st.nbytes > 0
        free0 = int(move.free_top.item())
        move.apply(leave=["b"])
        assert move.keys == ["a", "c"]
        assert int(move.free_top.item()) == free0 + (warm + 63) // 64
        other = model.make_cache(max_rows=2, n_pages=16, max_pages_per_row=4, seed=2)
        other.apply(join=[("b2", st)])
        assert other.host_pos() == [warm]
        for t in range(cont):
            want, _ = BT.forward(model, stay, cont_toks[t].tolist())
            got, _ = BT.forward(model, other, [int(cont_toks[t, 1])])
            assert torch.equal(got[0], want[1]), (mode, t)
            rest, _ = BT.forward(model, move, [int(cont_toks[t, 0]), int(cont_toks[t, 2])])
            assert torch.equal(rest[0], want[0]) and torch.equal(rest[1], want[2]), (mode, t)
        # a second capture of the moved row equals a capture of the row that stayed
        a, b = other.capture_row("b2"), stay.capture_row("b")
        assert a.pos == b.pos
        for ta, tb in zip(a.layers, b.layers):
            for xa, xb in zip(ta[1:], tb[1:]):
                if torch.is_tensor(xa):
                    assert torch.equal(xa, xb), (mode, ta[0])
                else:
                    assert xa == xb
    ops.check_status()
