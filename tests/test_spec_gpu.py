"""Batched verify + per-row commit (volundr_mlx_b200.batch_spec, after batch_spec.verify_forward / commit,
batch_spec.py:107-199) against plain sequential decoding: the T logits rows of every request equal those of feeding
its drafts one by one, and after commit(n_b) every request continues exactly like a request that only ever decoded its
first n_b drafts (own B = 1 cache), including a draft window that opens a new page which the commit has to hand back."""
import numpy as np
import pytest
import torch

from volundr_mlx_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda", 0)


@pytest.mark.parametrize("mode", ["reference", "paged_tokens"])
def test_verify_commit_equals_sequential_decode(cuda, mode):
    from volundr_mlx_b200 import batch as BT, batch_spec as SP, ops
    from volundr_mlx_b200.volundr import Model

    kw = {} if mode == "reference" else dict(bcsa_far="tokens", bcsa_score="pooled_key", bcsa_window=128,
                                             bcsa_compress=64, bcsa_topk=2)
    args = synth.small_args(**kw)
    params = synth.make_params(args, seed=12)
    model = Model(args, params, cuda)
    rng = np.random.default_rng(12)
    B, T, warm, cont = 3, 8, 60, 6           # drafts cover positions 60..67: a new page opens at 64
    warm_toks = rng.integers(0, args.vocab_valid, size=(warm, B))
    drafts = rng.integers(0, args.vocab_valid, size=(B, T))
    cont_toks = rng.integers(0, args.vocab_valid, size=(cont, B))
    accepted = [2, 8, 5]

    bc = model.make_cache(max_rows=4, n_pages=16, max_pages_per_row=4)
    bc.apply(join=["a", "b", "c"])
    for t in range(warm):
        BT.forward(model, bc, warm_toks[t].tolist())
    free_before = int(bc.free_top.item())
    logits, greedy, h = SP.verify_forward(model, bc, drafts.tolist())
    assert torch.equal(greedy.long(), logits.float()[:, :, : args.vocab_valid].argmax(dim=2))
    SP.commit(model, bc, h, accepted)
    assert bc.host_pos() == [warm + n for n in accepted]
    # rows that kept position 64 (n_b >= 5) hold one more page than before, the others gave theirs back
    assert int(bc.free_top.item()) == free_before - sum(1 for n in accepted if warm + n > 64)
    after = []
    for t in range(cont):
        lg, _ = BT.forward(model, bc, cont_toks[t].tolist())
        after.append(lg.clone())
    ops.check_status()

    for b in range(B):
        one = model.make_cache(max_rows=1, n_pages=8, max_pages_per_row=4)
        one.apply(join=["x"])
        for t in range(warm):
            BT.forward(model, one, [int(warm_toks[t, b])])
        seq = []
        for t in range(accepted[b]):
            lg, _ = BT.forward(model, one, [int(drafts[b, t])])
            seq.append(lg[0].clone())
        for t in range(accepted[b]):
            assert torch.equal(seq[t], logits[b, t]), (b, t)
        for t in range(cont):
            lg, _ = BT.forward(model, one, [int(cont_toks[t, b])])
            assert torch.equal(lg[0], after[t][b]), (b, t)
    ops.check_status()
