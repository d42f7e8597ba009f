"""T tokens per row in one pass over the weights (volundr_mlx_b200.chunk: the verify tile and the prefill chunk) against
token-by-token decoding of the same model: logits of every position, the state a commit leaves behind (checked through
the logits of the steps that follow) and the page accounting. Linears run with other row counts here than in the decode
step (other split of K over CTAs), so the comparison is at the bf16 floor, not bit for bit."""
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


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max())


@pytest.mark.parametrize("mode", ["reference", "paged_tokens"])
def test_verify_chunk_and_commit(cuda, mode):
    from volundr_mlx_b200 import batch as BT, chunk as CH, ops
    from volundr_mlx_b200.volundr import Model

    kw = {} if mode == "reference" else dict(bcsa_far="tokens", bcsa_score="pooled_key", bcsa_window=128,
                                             bcsa_compress=64, bcsa_topk=2)
    args = synth.small_args(**kw)
    params = synth.make_params(args, seed=31)
    model = Model(args, params, cuda)
    rng = np.random.default_rng(31)
    B, T, warm, cont = 3, 8, 60, 5           # the window covers positions 60..67: a page opens at 64
    warm_toks = rng.integers(0, args.vocab_valid, size=(warm, B))
    drafts = rng.integers(0, args.vocab_valid, size=(B, T))
    cont_toks = rng.integers(0, args.vocab_valid, size=(cont, B))
    accepted = [2, 8, 5]

    def fresh():
        bc = model.make_cache(max_rows=4, n_pages=16, max_pages_per_row=4)
        bc.apply(join=["a", "b", "c"])
        for t in range(warm):
            BT.forward(model, bc, warm_toks[t].tolist())
        return bc

    # sequential decoding of all T drafts: the logits the verify pass must reproduce
    seq = fresh()
    want = []
    for t in range(T):
        lg, _ = BT.forward(model, seq, drafts[:, t].tolist())
        want.append(lg.clone())
    want = torch.stack(want, dim=1)          # [B, T, V]

    bc = fresh()
    free_before = int(bc.free_top.item())
    logits, greedy, h = CH.forward_chunk(model, bc, drafts.tolist())
    ops.check_status()
    assert logits.shape == want.shape
    assert _rel(logits, want) < 3e-2
    assert torch.equal(greedy.long(), logits.float()[:, :, : args.vocab_valid].argmax(dim=2))
    CH.commit_chunk(model, bc, h, accepted)
    assert bc.host_pos() == [warm + n for n in accepted]
    assert int(bc.free_top.item()) == free_before - sum(1 for n in accepted if warm + n > 64)

    # every row must now continue like a request that decoded only its accepted drafts
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
        for t in range(accepted[b]):
            BT.forward(model, one, [int(drafts[b, t])])
        for t in range(cont):
            lg, _ = BT.forward(model, one, [int(cont_toks[t, b])])
            assert _rel(after[t][b], lg[0]) < 3e-2, (b, t)
    ops.check_status()


def test_prefill_chunks_then_decode(cuda):
    from volundr_mlx_b200 import batch as BT, chunk as CH, ops
    from volundr_mlx_b200.volundr import Model

    args = synth.small_args(bcsa_far="tokens", bcsa_score="pooled_key", bcsa_window=128, bcsa_compress=64, bcsa_topk=2)
    params = synth.make_params(args, seed=32)
    model = Model(args, params, cuda)
    rng = np.random.default_rng(32)
    prompt = rng.integers(0, args.vocab_valid, size=200).tolist()
    tail = rng.integers(0, args.vocab_valid, size=6).tolist()

    seq = model.make_cache(max_rows=1, n_pages=8, max_pages_per_row=6)
    seq.apply(join=["x"])
    want = []
    for t in prompt:
        lg, _ = BT.forward(model, seq, [t])
        want.append(lg[0].clone())

    bc = model.make_cache(max_rows=1, n_pages=8, max_pages_per_row=6)
    bc.apply(join=["x"])
    got = []
    for c0 in range(0, len(prompt), 48):     # chunks of 48 tokens (the last one shorter)
        lg, _, _ = CH.forward_chunk(model, bc, [prompt[c0:c0 + 48]], write=True)
        got.append(lg[0].clone())
    got = torch.cat(got)
    ops.check_status()
    assert bc.host_pos() == [len(prompt)]
    assert _rel(got, torch.stack(want)) < 3e-2
    for t in tail:
        a, _ = BT.forward(model, bc, [t])
        b, _ = BT.forward(model, seq, [t])
        assert _rel(a, b) < 3e-2
    ops.check_status()
    # logits_at: the LM head on one token of the chunk only gives that token's logits and greedy id
    two = [model.make_cache(max_rows=1, n_pages=8, max_pages_per_row=6) for _ in range(2)]
    for c in two:
        c.apply(join=["x"])
    full, gfull, _ = CH.forward_chunk(model, two[0], [prompt[:48]], write=True)
    full, gfull = full.clone(), gfull.clone()
    one, gone, _ = CH.forward_chunk(model, two[1], [prompt[:48]], write=True, logits_at=[30])
    ops.check_status()
    assert one.shape == (1, 1, full.shape[2]) and _rel(one[0, 0], full[0, 30]) < 1e-2   # (the LM head's row passes differ)
    assert int(gone[0, 0]) == int(one[0, 0, : args.vocab_valid].float().argmax())
    assert two[1].host_pos() == [48]


def test_ragged_chunk(cuda):
    """Rows that bring different numbers of tokens (1, 70 and 9: a decoding row beside two prompt rows, the long one
    crossing a page boundary and closing a block): the rows' tokens lie one after another, nothing is padded. The
    logits after each row's last token and the steps that follow must be those of token-by-token decoding; a ragged
    verify pass + commit must leave each row where its accepted count says."""
    from volundr_mlx_b200 import batch as BT, chunk as CH, ops
    from volundr_mlx_b200.volundr import Model

    args = synth.small_args(bcsa_far="tokens", bcsa_score="pooled_key", bcsa_window=128, bcsa_compress=64, bcsa_topk=2)
    params = synth.make_params(args, seed=33)
    model = Model(args, params, cuda)
    rng = np.random.default_rng(33)
    warm, lens, cont = 20, [1, 70, 9], 4
    warm_toks = rng.integers(0, args.vocab_valid, size=(warm, 3))
    toks = [rng.integers(0, args.vocab_valid, size=n).tolist() for n in lens]
    cont_toks = rng.integers(0, args.vocab_valid, size=(cont, 3))

    def fresh():
        bc = model.make_cache(max_rows=4, n_pages=16, max_pages_per_row=4)
        bc.apply(join=["a", "b", "c"])
        for t in range(warm):
            BT.forward(model, bc, warm_toks[t].tolist())
        return bc

    def solo(b, n_own):
        """Row b alone: warm-up, its first n_own chunk tokens; returns the cache and the last logits."""
        one = model.make_cache(max_rows=1, n_pages=8, max_pages_per_row=4)
        one.apply(join=["x"])
        lg = None
        for t in range(warm):
            lg, _ = BT.forward(model, one, [int(warm_toks[t, b])])
        for t in range(n_own):
            lg, _ = BT.forward(model, one, [int(toks[b][t])])
        return one, lg[0].clone()

    for accepted in (None, [1, 33, 0]):
        bc = fresh()
        free_before = int(bc.free_top.item())
        if accepted is None:
            logits, greedy, _ = CH.forward_chunk(model, bc, toks, write=True)
            kept = lens
        else:
            logits, greedy, h = CH.forward_chunk(model, bc, toks, write=False)
            CH.commit_chunk(model, bc, h, accepted)
            kept = accepted
        ops.check_status()
        assert logits.shape[:2] == (3, 1)
        assert bc.host_pos() == [warm + n for n in kept]
        assert int(bc.free_top.item()) == free_before - sum(1 for n in kept if warm + n > 64)
        after = []
        for t in range(cont):
            lg, _ = BT.forward(model, bc, cont_toks[t].tolist())
            after.append(lg.clone())
        ops.check_status()
        for b in range(3):
            one, last = solo(b, kept[b])
            if accepted is None:      # (the verify pass's logits follow the last token of the whole chunk row)
                assert _rel(logits[b, 0], last) < 3e-2, b
                assert int(greedy[b, 0]) == int(logits[b, 0, : args.vocab_valid].float().argmax())
            for t in range(cont):
                lg, _ = BT.forward(model, one, [int(cont_toks[t, b])])
                assert _rel(after[t][b], lg[0]) < 3e-2, (b, t, accepted)
    ops.check_status()
