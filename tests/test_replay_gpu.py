"""The captured step (one CUDA graph, every kernel launched with programmatic dependent launch, so that a kernel's
prologue runs beside its predecessor) against the same step launched kernel by kernel without it: bit for bit, every
step buffer, over enough steps that an ordering mistake between overlapped kernels shows.

What this guards: with dependent launch the KDA kernel's prologue (its loads of state, conv window and layer input)
runs beside the in_proj GEMM. That traffic once let a TMA refill of the GEMM's shared-memory ring land while a warp was
still reading the stage (the proxy fence between the producer's wait and its bulk copy was missing): a 32-row block of
the product came out wrong in every fourth step of this test."""
import numpy as np
import pytest
import torch

from oracle.model import Oracle
from volundr_mlx_b200 import synth

import seeding

pytestmark = pytest.mark.gpu

BUFFERS = ("x_in", "h", "proj", "mix", "r", "h2", "hn2", "gu", "mlp", "H", "hn", "logits")


@pytest.mark.parametrize("mixers,rows,steps", [(["kda"], 6, 80), (["kda", "bcsa", "kda", "attn"], 16, 24)])
def test_graph_replay_equals_serial_launches(cuda, mixers, rows, steps):
    from volundr_mlx_b200 import _lib, batch as BT, ops
    from volundr_mlx_b200.volundr import Model

    L = _lib.lib()
    args = synth.volundr32b_args(num_hidden_layers=len(mixers), mixer_types=mixers, engram_layers=[], engram_rows=1 << 12,
                                 vocab_size=4096, vocab_valid=4000)
    params = synth.make_params(args, seed=4, quant=True, bias_mode="minus8")
    model = Model(args, params, cuda)
    orc = Oracle(args, params, exact=False, w32=True)   # (only draws the rows' starting state)
    keys = list(range(rows))
    ctx = [300 + 37 * i for i in range(rows)]
    a, _ = seeding.seeded_batch(model, orc, keys, ctx, seed=4, max_rows=16, extra_tokens=steps + 8)
    b, _ = seeding.seeded_batch(model, orc, keys, ctx, seed=4, max_rows=16, extra_tokens=steps + 8)
    b.use_graph = False
    rng = np.random.default_rng(4)
    try:
        for t in range(steps):
            toks = rng.integers(0, args.vocab_valid, size=rows).tolist()
            L.vk_set_pdl(1)
            BT.forward(model, a, toks)
            torch.cuda.synchronize()
            L.vk_set_pdl(0)
            BT.forward(model, b, toks)
            torch.cuda.synchronize()
            for nm in BUFFERS:
                x, y = getattr(a, nm)[:rows], getattr(b, nm)[:rows]
                if not torch.equal(x, y):
                    cols = (x != y).nonzero()[:, -1].unique().tolist()
                    raise AssertionError(f"step {t}: {nm} differs between the graph replay and serial launches in "
                                         f"{len(cols)} columns, first {cols[:4]}")
    finally:
        L.vk_set_pdl(1)
    ops.check_status()
