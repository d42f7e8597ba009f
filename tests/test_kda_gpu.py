"""The KDA decode step as one operator (vk_kda_step through the C ABI) against the oracle's kda_core on the same
inputs: 40 value heads, d_k = d_v = 128, 16 rows, fp32 state N(0, 0.1), per-channel log-decay uniform in (-5, 0), beta =
sigmoid(N(0, 1)) (the third baseline configuration; the reference's layer, volundr.py:388-439). Bars: the fp32 state
within rtol 1e-4 / atol 1e-4 EVERYWHERE, the bf16 output within rtol 2e-2 / atol 2e-2.

The kernel forms in_proj_b, f_up and the causal conv itself and rounds them to bf16, so "the same inputs" needs care:
  * in_proj_b and f_up see one-hot inputs, so the products are single bf16 weights, exact on both sides; the weights
    are chosen to give the configuration's gate and beta distributions;
  * SiLU: expf on the device and np.exp differ in the last place, and a conv output whose SiLU falls that close to the
    midpoint of two bf16 values would round differently on the two sides. The newest input row is therefore redrawn,
    channel by channel, until no SiLU lies within 1e-5 (relative) of such a midpoint: both sides then hold the same
    post-SiLU q / k / v bits and the recurrence is compared on identical inputs.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle.model import Args, Oracle
from oracle.numerics import bf

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda", 0)


def _sparse_exact(rng, n, nnz):
    """n values, nnz of them +-2^e (e in -2..1), the rest zero: dot products with coarse weights are exact in fp32."""
    x = np.zeros(n, np.float32)
    idx = rng.choice(n, size=nnz, replace=False)
    x[idx] = rng.choice([-1.0, 1.0], size=nnz) * 2.0 ** rng.integers(-2, 2, size=nnz)
    return x


def _silu64(c):
    c = np.asarray(c, np.float64)
    return c / (1 + np.exp(-c))


def _near_bf16_tie(y, rel=1e-5, absolute=1e-6):
    """True where y lies within rel * |y| of the midpoint between two neighbouring bf16 values (where rounding to bf16
    could go either way under an error of that size; `absolute` covers the fp32 rounding of a conv sum whose terms cancel:
    a few 2^-24 of terms of order one). bf16 values of magnitude in [2^e, 2^(e+1)) are 2^(e-7) apart."""
    y = np.abs(np.asarray(y, np.float64))
    e = np.floor(np.log2(np.maximum(y, 1e-300)))
    step = np.exp2(e - 7)
    f = y / step
    f = f - np.floor(f)
    return np.abs(f - 0.5) * step < rel * y + absolute


def _taps(rng, C):
    """Conv taps N(0, 0.5) pushed away from zero (|w| >= 0.1): the newest input must be able to move every channel's
    conv output, or _draw_safe_row could not steer it clear of a rounding boundary."""
    w = rng.normal(0, 0.5, size=(C, 4))
    return bf(np.sign(w) * (0.1 + np.abs(w)))


def _draw_safe_row(rng, conv_prev, conv_w, n):
    """A new qkv row [C] (bf16 N(0, 1)) such that SiLU(conv) stays clear of every bf16 rounding boundary."""
    x = bf(rng.normal(0, 1, size=n))
    for _ in range(50):
        acc = conv_prev[0] * conv_w[:, 0]
        acc = acc + conv_prev[1] * conv_w[:, 1]
        acc = acc + conv_prev[2] * conv_w[:, 2]
        acc = (acc + x * conv_w[:, 3]).astype(np.float32)
        y = _silu64(acc)
        bad = _near_bf16_tie(y)
        if not bad.any():
            return x
        x = np.where(bad, bf(rng.normal(0, 1, size=n)), x)
    raise AssertionError("could not draw a row clear of the rounding boundaries")


@pytest.mark.parametrize("Hk", [40, 8])
def test_kda_step_state_and_output(cuda, Hk):
    from volundr_mlx_b200 import _lib, ops

    L = _lib.lib()
    rng = np.random.default_rng(2)
    B, HV, K, V, D, rank = 16, 40, 128, 128, 512, 64
    C = 2 * Hk * K + HV * V
    args = Args(linear_num_key_heads=Hk, linear_num_value_heads=HV, linear_key_head_dim=K, linear_value_head_dim=V,
                kda_gate_rank=rank)
    # row b feeds one-hot h = e_b and f_down = e_b: in_proj_b gives w_b[:, b] ~ N(0, 1) (beta = sigmoid of it), f_up
    # gives w_fup[:, b] = softplus^-1(d) with d ~ U(0, 5), so that with A_log = 0 and dt_bias = 0 the log-decay is -d
    w_b = bf(rng.normal(0, 1, size=(HV, D)))
    d = rng.uniform(1e-3, 5.0, size=(HV * K, rank))
    w_fup = bf(np.log(np.expm1(d)))
    conv_w = _taps(rng, C)
    A_log = np.zeros(HV, np.float32)
    dt_bias = np.zeros(HV * K, np.float32)
    norm_w = bf(1.0 + rng.normal(0, 0.1, size=V))
    params = {"l.conv1d.weight": conv_w, "l.A_log": A_log, "l.dt_bias": dt_bias, "l.norm.weight": norm_w}
    orc = Oracle(args, params, exact=False)

    ldp = C + HV * V + rank
    h = np.zeros((B, D), np.float32)
    h[np.arange(B), np.arange(B)] = 1.0
    S0 = rng.normal(0, 0.1, size=(B, HV, V, K)).astype(np.float32)
    conv0 = bf(rng.normal(0, 1, size=(B, 3, C)))

    bft = lambda x: torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(cuda).to(torch.bfloat16)
    f32 = lambda x: torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(cuda)
    t_h, t_wb = bft(h), bft(w_b)
    t_fup_rows = bft(w_fup)
    t_fup = torch.empty_like(t_fup_rows)
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(L.vk_kda_pack_fup(t_fup_rows.data_ptr(), t_fup.data_ptr(), HV, rank, st), "vk_kda_pack_fup")
    t_convw, t_alog, t_dtb, t_nw = f32(conv_w), f32(A_log), f32(dt_bias), bft(norm_w)
    t_conv = torch.zeros((2, B, 3, C), dtype=torch.bfloat16, device=cuda)
    t_conv[0] = bft(conv0)
    t_par = torch.zeros(1, dtype=torch.int32, device=cuda)
    t_S = f32(S0)
    t_out = torch.empty((B, HV * V), dtype=torch.bfloat16, device=cuda)
    _lib.check(L.vk_kda_configure(), "vk_kda_configure")

    steps = 3
    want_out = None
    rows = [{"conv": conv0[b].astype(np.float32).copy(), "S": S0[b].copy()} for b in range(B)]
    for s in range(steps):
        proj = np.zeros((B, ldp), np.float32)
        for b in range(B):
            proj[b, :C] = _draw_safe_row(rng, rows[b]["conv"], conv_w.astype(np.float32), C)
            proj[b, C + HV * V + b] = 1.0                                        # f_down = e_b
        proj[:, C: C + HV * V] = bf(rng.normal(0, 1, size=(B, HV * V)))          # z
        t_proj = bft(proj)
        _lib.check(L.vk_kda_step(t_proj.data_ptr(), ldp, C, C + HV * V, t_h.data_ptr(), t_wb.data_ptr(), t_fup.data_ptr(),
                                 t_convw.data_ptr(), t_alog.data_ptr(), t_dtb.data_ptr(), t_nw.data_ptr(), t_conv.data_ptr(),
                                 t_par.data_ptr(), t_conv[0].numel(), t_S.data_ptr(), t_out.data_ptr(), None, B, D, Hk,
                                 HV, K, V, rank, args.rms_norm_eps, st), "vk_kda_step")
        t_par ^= 1
        want_out = []
        for b in range(B):
            bdot = w_b[:, b]                                                     # the one-hot products, exact
            aa = w_fup[:, b].reshape(HV, K)
            z = proj[b, C: C + HV * V].reshape(HV, V)
            want_out.append(orc.kda_core("l.", proj[b, :C], z, bdot, aa, rows[b]))
    ops.check_status()

    got_S = t_S.cpu().numpy()
    want_S = np.stack([r["S"] for r in rows])
    np.testing.assert_allclose(got_S, want_S, rtol=1e-4, atol=1e-4)
    got = t_out.float().cpu().numpy().reshape(B, HV, V)
    np.testing.assert_allclose(got, np.stack(want_out), rtol=2e-2, atol=2e-2)
    # the conv state rolled forward: the buffer named by the parity word holds the last three inputs
    cur = int(t_par.item())
    got_conv = t_conv[cur].float().cpu().numpy()
    np.testing.assert_array_equal(got_conv, np.stack([r["conv"] for r in rows]))


def test_kda_chunk64_ragged_lengths_against_oracle(cuda):
    """The prefill form at chunk 64 over ragged prompt lengths (vk_kda_chunk_ragged, rows bring 64 tokens per launch and
    fewer in their last one) against the oracle's token-by-token recurrence: final fp32 state within 1e-4, every
    output within 2e-2. Lengths are a scaled-down draw of the configuration's log-uniform 256..20480 (the oracle walks
    them token by token); the full lengths are covered by the chunk kernel being bit-equal to single steps
    (test_kda_chunk_equals_steps) at any length."""
    from volundr_mlx_b200 import _lib, ops

    L = _lib.lib()
    rng = np.random.default_rng(22)
    B, Hk, HV, K, V, D, rank, T = 3, 8, 8, 128, 128, 64, 64, 64
    C = 2 * Hk * K + HV * V
    lengths = [int(x) for x in np.exp(rng.uniform(np.log(64), np.log(640), size=B))]
    lengths[0] = 257
    args = Args(linear_num_key_heads=Hk, linear_num_value_heads=HV, linear_key_head_dim=K, linear_value_head_dim=V,
                kda_gate_rank=rank)
    w_b = bf(rng.normal(0, 1, size=(HV, D)))
    w_fup = bf(np.log(np.expm1(rng.uniform(1e-3, 5.0, size=(HV * K, rank)))))
    conv_w = _taps(rng, C)
    A_log, dt_bias = np.zeros(HV, np.float32), np.zeros(HV * K, np.float32)
    norm_w = bf(1.0 + rng.normal(0, 0.1, size=V))
    params = {"l.conv1d.weight": conv_w, "l.A_log": A_log, "l.dt_bias": dt_bias, "l.norm.weight": norm_w}
    orc = Oracle(args, params, exact=False)
    ldp = C + HV * V + rank
    S0 = rng.normal(0, 0.1, size=(B, HV, V, K)).astype(np.float32)
    conv0 = bf(rng.normal(0, 1, size=(B, 3, C)))
    rows = [{"conv": conv0[b].astype(np.float32).copy(), "S": S0[b].copy()} for b in range(B)]
    # every token: one-hot h and f_down whose index cycles with the position (gates and beta change token by token)
    seqs, hs, wants = [], [], []
    for b in range(B):
        n = lengths[b]
        proj = np.zeros((n, ldp), np.float32)
        hrow = np.zeros((n, D), np.float32)
        outs = []
        win = rows[b]["conv"].copy()
        for t in range(n):
            x = _draw_safe_row(rng, win, conv_w.astype(np.float32), C)
            proj[t, :C] = x
            proj[t, C: C + HV * V] = bf(rng.normal(0, 1, size=HV * V))
            j = (t + 7 * b) % rank
            proj[t, C + HV * V + j] = 1.0
            hrow[t, (t + 3 * b) % D] = 1.0
            outs.append(orc.kda_core("l.", proj[t, :C], proj[t, C: C + HV * V].reshape(HV, V), w_b[:, (t + 3 * b) % D],
                                     w_fup[:, j].reshape(HV, K), rows[b]))
            win = np.concatenate([win[1:], x[None]])
        seqs.append(proj)
        hs.append(hrow)
        wants.append(np.stack(outs))

    bft = lambda x: torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(cuda).to(torch.bfloat16)
    f32 = lambda x: torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(cuda)
    st = torch.cuda.current_stream().cuda_stream
    t_wb, t_fup_rows = bft(w_b), bft(w_fup)
    t_fup = torch.empty_like(t_fup_rows)
    _lib.check(L.vk_kda_pack_fup(t_fup_rows.data_ptr(), t_fup.data_ptr(), HV, rank, st), "vk_kda_pack_fup")
    t_convw, t_alog, t_dtb, t_nw = f32(conv_w), f32(A_log), f32(dt_bias), bft(norm_w)
    t_conv = torch.zeros((2, B, 3, C), dtype=torch.bfloat16, device=cuda)
    t_conv[0] = bft(conv0)
    t_par = torch.zeros(1, dtype=torch.int32, device=cuda)
    t_S = f32(S0)
    _lib.check(L.vk_kda_configure(), "vk_kda_configure")
    got = [np.zeros((lengths[b], HV * V), np.float32) for b in range(B)]
    fed = [0] * B
    while any(fed[b] < lengths[b] for b in range(B)):
        n = [min(T, lengths[b] - fed[b]) for b in range(B)]
        # (a row that has finished still takes part with zero tokens: its state and conv window pass through)
        off = np.cumsum([0] + n[:-1]).astype(np.int32)
        R = int(sum(n))
        proj = np.concatenate([seqs[b][fed[b]: fed[b] + n[b]] for b in range(B)])
        hh = np.concatenate([hs[b][fed[b]: fed[b] + n[b]] for b in range(B)])
        t_proj, t_h = bft(proj), bft(hh)
        t_out = torch.zeros((R, HV * V), dtype=torch.bfloat16, device=cuda)
        t_acc = torch.tensor(n, dtype=torch.int32, device=cuda)
        t_off = torch.from_numpy(off).to(cuda)
        _lib.check(L.vk_kda_chunk_ragged(t_proj.data_ptr(), ldp, C, C + HV * V, t_h.data_ptr(), t_wb.data_ptr(), t_fup.data_ptr(),
                                         t_convw.data_ptr(), t_alog.data_ptr(), t_dtb.data_ptr(), t_nw.data_ptr(),
                                         t_conv.data_ptr(), t_par.data_ptr(), t_conv[0].numel(), t_S.data_ptr(), t_out.data_ptr(),
                                         t_acc.data_ptr(), t_off.data_ptr(), 1, B, T, D, Hk, HV, K, V, rank,
                                         args.rms_norm_eps, st), "vk_kda_chunk_ragged")
        t_par ^= 1
        o = t_out.float().cpu().numpy()
        for b in range(B):
            got[b][fed[b]: fed[b] + n[b]] = o[off[b]: off[b] + n[b]]
            fed[b] += n[b]
    ops.check_status()
    np.testing.assert_allclose(t_S.cpu().numpy(), np.stack([r["S"] for r in rows]), rtol=1e-4, atol=1e-4)
    for b in range(B):
        np.testing.assert_allclose(got[b].reshape(-1, HV, V), wants[b], rtol=2e-2, atol=2e-2)
    cur = int(t_par.item())
    np.testing.assert_array_equal(t_conv[cur].float().cpu().numpy(), np.stack([r["conv"] for r in rows]))


@pytest.mark.parametrize("Hk,T", [(40, 8), (8, 19)])
def test_kda_chunk_equals_steps(cuda, Hk, T):
    """vk_kda_chunk (T tokens per row in one launch: the prefill / verify form) against T calls of vk_kda_step on the
    same inputs: state, outputs and conv window bit for bit; with `accept`, row b equals accept[b] steps and its later
    outputs stay untouched (the commit replay of a verify step, batch_spec.py:186-195)."""
    from volundr_mlx_b200 import _lib, ops

    L = _lib.lib()
    g = torch.Generator(device="cpu").manual_seed(100 + T)
    B, HV, K, V, D, rank = 5, 40, 128, 128, 1024, 128
    C = 2 * Hk * K + HV * V
    ldp = C + HV * V + rank
    bf = dict(dtype=torch.bfloat16, device=cuda)
    proj = torch.randn(B, T, ldp, generator=g).to(**bf)
    h = torch.randn(B, T, D, generator=g).to(**bf)
    w_b = (torch.randn(HV, D, generator=g) * 0.05).to(**bf)
    fup_rows = (torch.randn(HV * K, rank, generator=g) * 0.1).to(**bf)
    fup = torch.empty_like(fup_rows)
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(L.vk_kda_pack_fup(fup_rows.data_ptr(), fup.data_ptr(), HV, rank, st), "vk_kda_pack_fup")
    conv_w = torch.randn(C, 4, generator=g).to(cuda)
    A_log = (torch.rand(HV, generator=g) * 2 - 1).to(cuda)
    dt_bias = torch.randn(HV * K, generator=g).to(cuda)
    norm_w = (1 + 0.1 * torch.randn(V, generator=g)).to(**bf)
    S0 = (torch.randn(B, HV, V, K, generator=g) * 0.1).to(cuda)
    conv0 = torch.randn(B, 3, C, generator=g).to(**bf)
    _lib.check(L.vk_kda_configure(), "vk_kda_configure")
    p = lambda t: t.data_ptr()

    def steps(n_per_row):
        """n_per_row[b] sequential vk_kda_step calls for row b (one row at a time)."""
        S, outs, convs = S0.clone(), torch.zeros(B, T, HV * V, **bf), torch.zeros(B, 3, C, **bf)
        for b in range(B):
            conv = torch.zeros(2, 1, 3, C, **bf)
            conv[0, 0] = conv0[b]
            par = torch.zeros(1, dtype=torch.int32, device=cuda)
            Sb = S[b:b + 1].clone()
            for t in range(n_per_row[b]):
                o = torch.empty(1, HV * V, **bf)
                _lib.check(L.vk_kda_step(p(proj[b, t]), ldp, C, C + HV * V, p(h[b, t]), p(w_b), p(fup), p(conv_w), p(A_log),
                                         p(dt_bias), p(norm_w), p(conv), p(par), conv[0].numel(), p(Sb), p(o), None, 1,
                                         D, Hk, HV, K, V, rank, 1e-6, st), "vk_kda_step")
                par ^= 1
                outs[b, t] = o[0]
            S[b] = Sb[0]
            convs[b] = conv[int(par.item()), 0]
        return S, outs, convs

    def chunk(accept):
        S, outs = S0.clone(), torch.zeros(B, T, HV * V, **bf)
        conv = torch.zeros(2, B, 3, C, **bf)
        conv[0] = conv0
        par = torch.zeros(1, dtype=torch.int32, device=cuda)
        acc = torch.tensor(accept, dtype=torch.int32, device=cuda) if accept is not None else None
        _lib.check(L.vk_kda_chunk(p(proj), ldp, C, C + HV * V, p(h), p(w_b), p(fup), p(conv_w), p(A_log), p(dt_bias),
                                  p(norm_w), p(conv), p(par), conv[0].numel(), p(S), p(outs), p(acc) if acc is not None else None,
                                  1, B, T, D, Hk, HV, K, V, rank, 1e-6, st), "vk_kda_chunk")
        return S, outs, conv[1]

    for accept in (None, [0, 1, T // 2, T - 1, T]):
        want = steps([T] * B if accept is None else accept)
        got = chunk(accept)
        ops.check_status()
        for name, a, b_ in zip(("state", "out", "conv"), got, want):
            assert torch.equal(a, b_), (name, accept, float((a.float() - b_.float()).abs().max()))
