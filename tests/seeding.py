"""Rows that already hold a context, with the same state on the GPU cache and in the CPU oracle.

BASELINE's configurations start from rows with hundreds to thousands of tokens of context (bf16 K/V ~ N(0, 1), fp32 KDA
state ~ N(0, 0.1)). Decoding that many tokens through the oracle first would take hours, so the state is drawn
directly: one seeded draw fills an oracle `Row` and a `session.State`, and the State joins the batch through
`BatchCache.apply(join=[(key, state)])` (which scatters it into pages from the shuffled pool). Pooled block means are
formed by the oracle's own `pool` arithmetic (volundr.py:470-476) from the drawn K/V, so both sides select far blocks
from identical bits."""
import numpy as np
import torch

from oracle.numerics import bf


def _pool_blocks(x, C):
    """x [P, ...] bf16-valued float32 -> [P // C, ...]: rows of a block added in order in float32, times 1/C, one
    rounding (Oracle.pool)."""
    nb = x.shape[0] // C
    if nb == 0:
        return np.zeros((0,) + x.shape[1:], np.float32)
    blk = x[: nb * C].reshape((nb, C) + x.shape[1:])
    acc = np.zeros((nb,) + x.shape[1:], np.float32)
    for c in range(C):
        acc = (acc + blk[:, c]).astype(np.float32)
    return bf(acc * np.float32(1.0 / C))


def draw_row(args, orc, P, rng, device):
    """One sequence holding P tokens: returns (oracle Row, session.State on `device`)."""
    from volundr_mlx_b200 import session as SS

    a = args
    row = orc.new_row()
    row.pos = P
    layers = []
    KVH, D = a.num_key_value_heads, a.head_dim
    Cc = 2 * a.linear_num_key_heads * a.linear_key_head_dim + a.linear_num_value_heads * a.linear_value_head_dim
    bft = lambda x: torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(device).to(torch.bfloat16)
    f32 = lambda x: torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(device)
    for i, m in enumerate(a.mixer_types):
        st = row.layers[i]
        if m == "kda":
            conv = bf(rng.normal(0, 1, size=(3, Cc)))
            S = rng.normal(0, 0.1, size=(a.linear_num_value_heads, a.linear_value_head_dim, a.linear_key_head_dim)).astype(np.float32)
            st["conv"], st["S"] = conv.copy(), S.copy()
            layers.append(("arrays", bft(conv)[None], f32(S)[None]))
            continue
        K = bf(rng.normal(0, 1, size=(P, KVH, D)))
        V = bf(rng.normal(0, 1, size=(P, KVH, D)))
        st["k"], st["v"] = list(K), list(V)
        kt, vt = bft(K.transpose(1, 0, 2))[None], bft(V.transpose(1, 0, 2))[None]
        if m == "attn":
            layers.append(("kv", P, kt, vt))
            continue
        C = a.bcsa_compress
        nb = P // C
        PK, PV = _pool_blocks(K, C), _pool_blocks(V, C)
        st["pk"], st["pv"] = list(PK), list(PV)
        bk_t = ik_t = None
        if a.bcsa_score == "indexer":
            Di = a.bcsa_index_dim
            BK = bf(rng.normal(0, 1, size=(nb, Di)))
            st["bk"] = list(BK)
            ik = np.zeros((C, Di), np.float32)
            for t in range(nb * C, P):          # the open block's keys, slot = position % C
                ik[t % C] = bf(rng.normal(0, 1, size=Di))
                st["ik_open"][t % C] = ik[t % C].copy()
            bk_t, ik_t = bft(BK)[None], bft(ik)[None]
        layers.append(("bcsa", a.bcsa_window, C, 0, P, nb, kt, vt, bft(PK.transpose(1, 0, 2))[None],
                       bft(PV.transpose(1, 0, 2))[None], bk_t, ik_t))
    keep = max(a.engram_orders) - 1 if a.engram_layers else 0
    prev = [int(x) for x in rng.integers(0, a.vocab_valid, size=keep)]
    row.prev = list(prev)
    layers.append(("engram", keep, torch.tensor([prev], dtype=torch.int32, device=device).reshape(1, keep)))
    state = SS.State(P, layers)
    state.count_bytes()
    return row, state


def seeded_batch(model, orc, keys, ctx_lens, seed, n_pages=None, max_rows=None, extra_tokens=64):
    """A BatchCache whose rows `keys` hold ctx_lens[i] tokens each, and the oracle rows with the same state."""
    args = model.args
    rng = np.random.Generator(np.random.PCG64(seed))
    pages_row = max((c + extra_tokens) // 64 + 2 for c in ctx_lens)
    n_pages = n_pages or sum((c + extra_tokens) // 64 + 2 for c in ctx_lens) + 4
    bc = model.make_cache(max_rows=max_rows or max(len(keys), 1), n_pages=n_pages, max_pages_per_row=pages_row, seed=seed)
    rows = {}
    join = []
    for k, P in zip(keys, ctx_lens):
        rows[k], st = draw_row(args, orc, int(P), rng, model.device)
        join.append((k, st))
    bc.apply(join=join)
    return bc, rows


def seeded_rows(model, orc, ctx_lens, keys, seed):
    """The oracle rows seeded_batch(model, ., keys, ctx_lens, seed) draws, for another oracle object (same values)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    return {k: draw_row(model.args, orc, int(P), rng, model.device)[0] for k, P in zip(keys, ctx_lens)}


def _close(got, want, tol, what):
    """Element-wise within tol * (|want| + the tensor's scale): values that went through several layers of bf16 arithmetic
    agree to a fraction of the vector's scale, not of each (possibly tiny) element."""
    want = np.asarray(want, np.float32)
    scale = float(np.abs(want).max()) if want.size else 0.0
    np.testing.assert_allclose(got, want, rtol=tol, atol=tol * max(scale, 1e-6), err_msg=str(what))


def assert_state_close(bc, key, row, args, s_atol=2e-3, tol=2e-2, what="", layers=None):
    """The cache row `key` (through BatchCache.capture_row) against the oracle's Row: position and Engram ids exactly;
    K / V by position, pooled block means, pooled and open-block indexer keys and the conv window within the bf16 bar
    (rtol = tol, atol = tol x the tensor's largest magnitude: the two sides hold bf16 roundings of hidden states that
    agree to a fraction of a percent of their scale after a few layers); the fp32 KDA state within s_atol for all but
    one element in 1e5, those within ten times that (its inputs carry that bf16-level noise; the 1e-4 bar on identical
    inputs is tests/test_kda_gpu.py's)."""
    st = bc.capture_row(key)
    a = args
    assert st.pos == row.pos, (what, st.pos, row.pos)
    P = row.pos
    f = lambda t: t.float().cpu().numpy()
    for i, (m, t) in enumerate(zip(a.mixer_types, st.layers)):
        o = row.layers[i]
        tag = (what, "layer", i, m)
        if layers is not None and i not in layers:
            continue
        if m == "kda":
            _close(f(t[1])[0], o["conv"], tol, tag + ("conv",))
            got_s, want_s = f(t[2])[0], np.asarray(o["S"], np.float32)
            out = np.abs(got_s - want_s) > s_atol + 1e-3 * np.abs(want_s)
            # (one bf16 step in one of a step's q / k / v inputs, 2^-8 of its magnitude, moves single elements of the
            # state by a few 1e-3: a handful of elements may sit there, none further out)
            assert out.mean() <= 1e-5, tag + ("S", float(out.mean()))
            np.testing.assert_allclose(got_s, want_s, rtol=1e-3, atol=10 * s_atol, err_msg=str(tag + ("S",)))
            continue
        k, v = (t[2], t[3]) if m == "attn" else (t[6], t[7])
        _close(f(k)[0], np.stack(o["k"]).transpose(1, 0, 2), tol, tag + ("K",))
        _close(f(v)[0], np.stack(o["v"]).transpose(1, 0, 2), tol, tag + ("V",))
        if m == "bcsa":
            C = a.bcsa_compress
            nb = P // C
            assert t[5] == nb == len(o["pk"]), tag
            if nb:
                _close(f(t[8])[0], np.stack(o["pk"]).transpose(1, 0, 2), tol, tag + ("PK",))
                _close(f(t[9])[0], np.stack(o["pv"]).transpose(1, 0, 2), tol, tag + ("PV",))
            if a.bcsa_score == "indexer":
                if nb:
                    _close(f(t[10])[0], np.stack(o["bk"]), tol, tag + ("BK",))
                ik = f(t[11])[0]
                assert sorted(o["ik_open"]) == [p % C for p in range(nb * C, P)], tag
                for slot, want in o["ik_open"].items():
                    _close(ik[slot], want, tol, tag + ("IK", slot))
    assert f(st.layers[-1][2])[0].astype(np.int64).tolist() == [int(x) for x in row.prev], (what, "engram ids")
