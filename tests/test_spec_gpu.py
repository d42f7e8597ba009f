"""Batched verify + per-row commit with the reference's signatures (batch_spec.verify_forward(model, bc, ids, capture) ->
(logits, features, rec); batch_spec.commit(bc, rec, ns); batch_spec.py:107-128, :173-199) against the CPU oracle, at the
block / window phases the reference's own test walks (tests/test_batch.py:180-219: rows starting at ([3, 0, 9],
[15, 22, 40], [1, 2, 3], [60, 7, 13]) with W = 16, C = 4, top-k 3, so that verify windows start inside a block, straddle
the window's fill-up, close several blocks and open a page): after commit(ns) every row must hold exactly what
sequential decoding of its first ns[b] tokens leaves (cache state compared with the oracle's row), and go on decoding
like it."""
import copy

import numpy as np
import pytest
import torch

from oracle.model import Oracle
from volundr_mlx_b200 import synth

import seeding

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("starts", [[3, 0, 9], [15, 22, 40], [1, 2, 3], [60, 7, 13]])
def test_verify_commit_at_block_and_window_phases(cuda, starts):
    from volundr_mlx_b200 import batch as BT, batch_spec as SP, ops
    from volundr_mlx_b200.volundr import Model

    args = synth.small_args()                     # the reference form: W = 16, C = 4, top-k 3, shared indexer
    params = synth.make_params(args, seed=12)
    model = Model(args, params, cuda)
    orc = Oracle(args, params, exact=False)
    rng = np.random.default_rng(sum(starts))
    keys = ["a", "b", "c"]
    T, cont = 6, 22
    bc = model.make_cache(max_rows=4, n_pages=16, max_pages_per_row=4)
    rows = {k: orc.new_row() for k in keys}
    # rows join late enough to stand at their start positions together
    top = max(starts)
    for t in range(top):
        join = [k for k, s in zip(keys, starts) if top - s == t]
        if join:
            bc.apply(join=join)
        if bc.B:
            toks = rng.integers(0, args.vocab_valid, size=bc.B).tolist()
            BT.forward(model, bc, toks)
            for r, k in enumerate(bc.keys):
                orc.step(rows[k], toks[r])
    late = [k for k in keys if k not in bc.keys]
    if late:
        bc.apply(join=late)
    order = list(bc.keys)
    assert bc.host_pos() == [starts[keys.index(k)] for k in order]

    for rnd in range(2):                          # two verify / commit rounds in a row
        ids = rng.integers(0, args.vocab_valid, size=(3, T))
        ns = [int(x) for x in rng.integers(1, T + 1, size=3)]
        before = bc.host_pos()
        logits, feats, rec = SP.verify_forward(model, bc, ids.tolist(), capture=())
        assert feats is None and bc.host_pos() == before
        got = logits.float().cpu().numpy()
        for r, k in enumerate(order):
            probe = copy.deepcopy(rows[k])
            for t in range(T):
                np.testing.assert_allclose(got[r, t], orc.step(probe, int(ids[r, t])), rtol=2e-2, atol=2e-2,
                                           err_msg=str((starts, rnd, k, t)))
        SP.commit(bc, rec, ns)
        for r, k in enumerate(order):
            for t in range(ns[r]):
                orc.step(rows[k], int(ids[r, t]))
        assert bc.host_pos() == [p + n for p, n in zip(before, ns)]
        ops.check_status()
        for k in order:
            seeding.assert_state_close(bc, k, rows[k], args, what=(starts, rnd, k))
    for t in range(cont):
        toks = rng.integers(0, args.vocab_valid, size=3).tolist()
        lg, _ = BT.forward(model, bc, toks)
        got = lg.float().cpu().numpy()
        for r, k in enumerate(order):
            np.testing.assert_allclose(got[r], orc.step(rows[k], toks[r]), rtol=2e-2, atol=2e-2, err_msg=str((starts, "after", t, k)))
    ops.check_status()
