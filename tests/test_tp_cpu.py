"""The multi-rank logic on CPU (gloo, world size 2): the tensor-parallel split of every linear (heads, MLP columns,
vocabulary) reproduces the unsplit layer after the all-reduce that the GPU path performs after out_proj / o_proj and
down_proj, and the sharded greedy token equals the first maximum of the full logits."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from volundr_mlx_b200 import sharding, synth


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        a = synth.small_args(num_attention_heads=8, num_key_value_heads=4, linear_num_key_heads=2, linear_num_value_heads=4)
        p = synth.make_params(a, seed=2, quant=False, dtype_round=False)
        rng = np.random.default_rng(0)
        B = 3
        h = rng.normal(size=(B, a.hidden_size))
        sharding.check(a, world)

        def allreduce(x):
            t = torch.from_numpy(np.ascontiguousarray(x))
            dist.all_reduce(t)
            return t.numpy()

        err = 0.0
        # MLP: column-parallel gate / up, row-parallel down
        L = "model.layers.0.mlp."
        sm = sharding.mlp_rows(a, rank, world)
        g, u = h @ p[L + "gate_proj.weight"][sm["gate"]].T, h @ p[L + "up_proj.weight"][sm["up"]].T
        act = g / (1 + np.exp(-g)) * u
        c0, c1 = sm["down_cols"]
        got = allreduce(act @ p[L + "down_proj.weight"][:, c0:c1].T)
        gf, uf = h @ p[L + "gate_proj.weight"].T, h @ p[L + "up_proj.weight"].T
        want = (gf / (1 + np.exp(-gf)) * uf) @ p[L + "down_proj.weight"].T
        err = max(err, np.abs(got - want).max() / np.abs(want).max())
        # KDA projections: the rank's q | k | v rows are whole heads, and value head hv still finds its key head
        sh = sharding.kda_rows(a, rank, world)
        K = a.linear_key_head_dim
        Hk, HV = a.linear_num_key_heads // world, a.linear_num_value_heads // world
        qkv_full = h @ p["model.layers.0.linear_attn.in_proj_qkv.weight"].T
        qkv_loc = h @ p["model.layers.0.linear_attn.in_proj_qkv.weight"][sh["qkv"]].T
        kd = a.linear_num_key_heads * K
        rep_full = a.linear_num_value_heads // a.linear_num_key_heads
        for hv_loc in range(HV):
            hv = rank * HV + hv_loc
            hk_loc = hv_loc // (HV // Hk)
            assert rank * Hk + hk_loc == hv // rep_full
            assert np.array_equal(qkv_loc[:, hk_loc * K:(hk_loc + 1) * K], qkv_full[:, (hv // rep_full) * K:(hv // rep_full + 1) * K])
            assert np.array_equal(qkv_loc[:, 2 * Hk * K + hv_loc * K: 2 * Hk * K + (hv_loc + 1) * K],
                                  qkv_full[:, 2 * kd + hv * K: 2 * kd + (hv + 1) * K])
        o0, o1 = sh["out_cols"]
        mix = rng.normal(size=(B, a.linear_num_value_heads * a.linear_value_head_dim))  # same on both ranks (seeded)
        got = allreduce(mix[:, o0:o1] @ p["model.layers.0.linear_attn.out_proj.weight"][:, o0:o1].T)
        want = mix @ p["model.layers.0.linear_attn.out_proj.weight"].T
        err = max(err, np.abs(got - want).max() / np.abs(want).max())
        # attention: q rows keep the per-head [q | gate] interleave
        sa = sharding.attn_rows(a, rank, world)
        D, Hq = a.head_dim, a.num_attention_heads // world
        qf = (h @ p["model.layers.2.self_attn.q_proj.weight"].T).reshape(B, a.num_attention_heads, 2 * D)
        ql = (h @ p["model.layers.2.self_attn.q_proj.weight"][sa["q"]].T).reshape(B, Hq, 2 * D)
        assert np.array_equal(ql, qf[:, rank * Hq:(rank + 1) * Hq])
        # vocabulary-sharded greedy token: ties to the lowest index
        v0, v1 = sharding.vocab_rows(a, rank, world)
        logits = np.round(rng.normal(size=(B, a.vocab_size)) * 2) / 2          # coarse: many ties
        logits[0, [5, v1 - 1 if rank == 0 else 7]] = 99.0
        valid = max(0, min(a.vocab_valid - v0, v1 - v0))
        loc = logits[:, v0:v0 + valid]
        vals = torch.from_numpy(loc.max(1)) if valid else torch.full((B,), -np.inf, dtype=torch.float64)
        idxs = torch.from_numpy(loc.argmax(1) + v0) if valid else torch.full((B,), 2 ** 31 - 1, dtype=torch.int64)
        gv = [torch.zeros_like(vals) for _ in range(world)]
        gi = [torch.zeros_like(idxs) for _ in range(world)]
        dist.all_gather(gv, vals)
        dist.all_gather(gi, idxs)
        tok = sharding.merge_argmax(torch.stack(gv).numpy(), torch.stack(gi).numpy())
        # every rank drew the same logits except the planted ties; compare on rank 0's copy
        full = torch.from_numpy(logits)
        dist.broadcast(full, 0)
        if rank == 0:
            pass
        out.put((rank, float(err), tok.tolist(), full[:, : a.vocab_valid].numpy().argmax(1).tolist() if rank == 0 else None))
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_split_world2():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, tok, want in res:
        assert err < 1e-12, (rank, err)
    # rows 1.. of the logits are identical on both ranks, so the merged token must be the full row's first maximum
    assert res[0][2][1:] == res[0][3][1:] == res[1][2][1:]


def test_merge_argmax_ties():
    vals = np.array([[1.0, 3.0], [1.0, 2.0]])
    idxs = np.array([[7, 4], [3, 9]])
    assert sharding.merge_argmax(vals, idxs).tolist() == [3, 4]


def test_peer_handle_layout():
    from volundr_mlx_b200 import peer

    hs = [bytes([r]) * 64 for r in range(4)]
    for r in range(4):
        lay = peer.handle_layout(4, r, hs)
        assert lay[r] is None and [h for h in lay if h is not None] == [hs[p] for p in range(4) if p != r]
    with pytest.raises(ValueError):
        peer.handle_layout(4, 0, hs[:3])
    with pytest.raises(ValueError):
        peer.handle_layout(2, 0, [b"x" * 63, b"y" * 64])
