"""The batched decode step on the GPU (through the C ABI, behind the reference's batch API) against the CPU oracle
row by row: every row of a ragged batch must reproduce its own B = 1 oracle run (the reference's test_batch.py:49-116
pins "each row == its own B = 1 run"; test_volundr.py:301-317 gives the bf16 bar: error at the bf16 floor of the
model and argmax agreement >= 90 %)."""
import numpy as np
import pytest
import torch

from oracle.model import Oracle
from volundr_mlx_b200 import synth

pytestmark = pytest.mark.gpu


def run_schedule(model, bc, orc, args, joins, leaves, steps, seed, BT):
    """Teacher-forced decode: row i joins at step joins[i] and leaves after leaves[i] tokens (test_batch.py:77-101)."""
    rng = np.random.default_rng(seed)
    n = len(joins)
    feeds = {i: rng.integers(0, args.vocab_valid, size=steps).tolist() for i in range(n)}
    rows = {i: orc.new_row() for i in range(n)}
    fed = {i: 0 for i in range(n)}
    worst, agree, total = 0.0, 0, 0
    for t in range(steps):
        join = [i for i in range(n) if joins[i] == t]
        leave = [i for i in list(bc.keys) if fed[i] >= leaves[i]]
        if join or leave:
            bc.apply(leave=leave, join=join)
        if not bc.B:
            continue
        toks = [feeds[i][fed[i]] for i in bc.keys]
        logits, _ = BT.forward(model, bc, toks)
        got = logits.float().cpu().numpy()
        greedy = bc.greedy[: bc.B].cpu().numpy()
        for r, i in enumerate(bc.keys):
            want = orc.step(rows[i], toks[r])
            fed[i] += 1
            err = np.abs(got[r] - want).max() / np.abs(want).max()
            worst = max(worst, err)
            v = args.vocab_valid
            assert greedy[r] == int(np.argmax(got[r][:v])), "device argmax is the first maximum over the valid vocabulary"
            total += 1
            # tie-aware agreement: the device's choice is within rounding of the oracle's best logit
            best = want[:v].max()
            agree += int(want[greedy[r]] >= best - 0.02 * np.abs(want).max())
        assert bc.host_pos() == [rows[i].pos for i in bc.keys]
    return worst, agree / total


@pytest.mark.parametrize("mode", ["reference", "paged_tokens"])
def test_rows_match_their_own_b1_oracle(cuda, mode):
    from volundr_mlx_b200 import batch as BT
    from volundr_mlx_b200.volundr import Model

    kw = {} if mode == "reference" else dict(bcsa_far="tokens", bcsa_score="pooled_key", bcsa_window=128,
                                             bcsa_compress=64, bcsa_topk=2)
    args = synth.small_args(**kw)
    params = synth.make_params(args, seed=3, quant=True, bias_mode="minus8")
    model = Model(args, params, cuda)
    orc = Oracle(args, params, exact=False)
    bc = model.make_cache(max_rows=8, n_pages=64, max_pages_per_row=8)
    steps = 60 if mode == "reference" else 330
    joins = [0, 0, 2, 3, 5] if mode == "reference" else [0, 0, 40]
    leaves = [60, 25, 50, 12, 40] if mode == "reference" else [330, 200, 280]
    worst, agree = run_schedule(model, bc, orc, args, joins, leaves, steps, 7, BT)
    from volundr_mlx_b200 import ops
    ops.check_status()
    assert worst < 5e-2, worst
    assert agree >= 0.97, agree


def test_graph_replay_equals_eager(cuda):
    """The CUDA-graph replay of a step gives the same logits, bit for bit, as launching the kernels one by one."""
    from volundr_mlx_b200 import batch as BT
    from volundr_mlx_b200.volundr import Model

    args = synth.small_args()
    params = synth.make_params(args, seed=5)
    model = Model(args, params, cuda)
    outs = []
    for use_graph in (True, False):
        bc = model.make_cache(max_rows=4, n_pages=32, max_pages_per_row=4)
        bc.use_graph = use_graph
        bc.apply(join=["a", "b", "c"])
        rng = np.random.default_rng(0)
        res = []
        for t in range(40):
            lg, _ = BT.forward(model, bc, rng.integers(0, args.vocab_valid, size=3).tolist())
            res.append(lg.clone())
        outs.append(torch.stack(res))
    assert torch.equal(outs[0], outs[1])


def test_fused_layer_boundary_equals_separate_kernels(cuda):
    """combine(i) + mix(i + 1) in one kernel gives the same logits, bit for bit, as the separate kernels."""
    from volundr_mlx_b200 import batch as BT
    from volundr_mlx_b200.volundr import Model

    args = synth.small_args()
    params = synth.make_params(args, seed=6)
    model = Model(args, params, cuda)
    outs = []
    for fuse in (True, False):
        bc = model.make_cache(max_rows=4, n_pages=32, max_pages_per_row=4)
        bc.fuse_boundary = fuse
        bc.apply(join=["a", "b", "c"])
        rng = np.random.default_rng(1)
        res = []
        for t in range(30):
            lg, _ = BT.forward(model, bc, rng.integers(0, args.vocab_valid, size=3).tolist())
            res.append(lg.clone())
        outs.append(torch.stack(res))
    assert torch.equal(outs[0], outs[1])


def test_clustered_boundary_close_to_single_cta(cuda):
    """A cluster of four CTAs per row in the layer-boundary kernel (hidden sizes that are multiples of 1024) adds the
    row-wide sums in another order than the one-CTA kernel: logits within the bf16 floor of each other, and each
    variant reproducible bit for bit."""
    from volundr_mlx_b200 import _lib, batch as BT
    from volundr_mlx_b200.volundr import Model

    L = _lib.lib()
    args = synth.block2_args()
    assert args.hidden_size % 1024 == 0
    params = synth.make_params(args, seed=11)
    model = Model(args, params, cuda)
    outs = []
    try:
        for cluster in (1, 0, 1):
            L.vk_mhc_boundary_set_cluster(cluster)
            bc = model.make_cache(max_rows=4, n_pages=32, max_pages_per_row=4)
            bc.apply(join=["a", "b", "c"])
            rng = np.random.default_rng(5)
            res = []
            for t in range(40):
                lg, _ = BT.forward(model, bc, rng.integers(0, args.vocab_valid, size=3).tolist())
                res.append(lg.float().clone())
            outs.append(torch.stack(res))
    finally:
        L.vk_mhc_boundary_set_cluster(0)
    from volundr_mlx_b200 import ops
    ops.check_status()
    assert torch.equal(outs[0], outs[2])
    scale = outs[1].abs().max()
    assert float((outs[0] - outs[1]).abs().max() / scale) < 3e-2


def test_tensor_core_attention_close_to_scalar_kernel(cuda):
    """The tensor-core attention (bf16 probabilities) against the scalar fp32 kernel on the same schedule: logits
    within bf16 tolerance (the reference's bar for its attention kernels is 2^-7 |x| + 2e-3, test_volundr.py:266)."""
    from volundr_mlx_b200 import _lib, batch as BT
    from volundr_mlx_b200.volundr import Model

    L = _lib.lib()
    args = synth.small_args(bcsa_far="tokens", bcsa_score="pooled_key", bcsa_window=128, bcsa_compress=64, bcsa_topk=2)
    params = synth.make_params(args, seed=8)
    model = Model(args, params, cuda)
    outs = []
    try:
        for tc in (1, 0):
            L.vk_attend_set_tensor_cores(tc)
            bc = model.make_cache(max_rows=4, n_pages=64, max_pages_per_row=8)
            bc.use_graph = False
            bc.apply(join=["a", "b"])
            rng = np.random.default_rng(2)
            res = []
            for t in range(300):
                lg, _ = BT.forward(model, bc, rng.integers(0, args.vocab_valid, size=2).tolist())
                if t % 10 == 9:
                    res.append(lg.float().clone())
            outs.append(torch.stack(res))
    finally:
        L.vk_attend_set_tensor_cores(1)
    err = (outs[0] - outs[1]).abs().max() / outs[1].abs().max()
    assert err < 2e-2, float(err)
