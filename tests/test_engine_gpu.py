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
