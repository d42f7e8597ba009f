"""W4 affine GEMM / dequant on the GPU against the CPU oracle (oracle/w4.py), called through the C ABI.
Shapes follow the W4A16 small-M sweep (M in {1,2,4,8,16}, K = 5120, N in {5120, 22016, 44032}), codes uniform in
[0,15], scales |N(0,0.02)|/8, biases N(0,0.01), activations N(0,1). Tolerance rtol 2e-2 / atol 2e-2 (bf16 outputs,
fp32 accumulation); dequantised weights bit-exact."""
import numpy as np
import pytest
import torch

from oracle import w4 as OW
from oracle.numerics import bf, bf_bits

pytestmark = pytest.mark.gpu


def make_w4(rng, N, K, group, bias_mode="free"):
    u = rng.integers(0, 16, size=(N, K))
    s = bf(np.abs(rng.normal(0, 0.02, size=(N, K // group))) / 8)
    if bias_mode == "free":
        b = bf(rng.normal(0, 0.01, size=(N, K // group)))
    else:  # the converter's case: bias = -8 scale (exact in bf16)
        b = bf(-8.0 * s)
    return OW.pack_codes(u), s, b


def to_dev(w, s, b, dev):
    tw = torch.from_numpy(w.view(np.int32)).to(dev)
    ts = torch.from_numpy(s).to(dev).to(torch.bfloat16)
    tb = torch.from_numpy(b).to(dev).to(torch.bfloat16)
    return tw, ts, tb


def bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("group,bias_mode", [(64, "free"), (128, "free"), (64, "minus8"), (128, "minus8")])
def test_dequant_bit_exact(cuda, group, bias_mode):
    from volundr_mlx_b200 import ops

    rng = np.random.default_rng(11)
    N, K = 96, 1024
    w, s, b = make_w4(rng, N, K, group, bias_mode)
    # tiny and zero biases exercise the single-rounding definition
    if bias_mode == "free":
        b[0, :4] = bf(np.array([0.0, 1e-30, -1e-12, 3e-9], dtype=np.float32))
    got = ops.w4_dequant(*to_dev(w, s, b, cuda), group)
    want = OW.dequant(w, s, b, group)
    assert np.array_equal(bits(got), bf_bits(want))
    if bias_mode == "minus8":  # the reference's pinned case: dequant == bf16(q * scale), q = u - 8
        q = OW.unpack_codes(w, K).astype(np.float32) - 8
        assert np.array_equal(bf_bits(want), bf_bits(bf(q * np.repeat(s, group, axis=1))))


def _check_gemm(cuda, rng, M, N, K, group, cols=None, force=None):
    from volundr_mlx_b200 import _lib, ops

    w, s, b = make_w4(rng, N, K, group)
    x = bf(rng.normal(0, 1, size=(M, K)))
    wt = ops.w4_repack(*to_dev(w, s, b, cuda), group)
    tx = torch.from_numpy(x).to(cuda).to(torch.bfloat16)
    L = _lib.lib()
    sel = np.arange(N) if cols is None else cols
    want = OW.matmul(x, w[sel], s[sel], b[sel], group)
    W = OW.unpack_codes(w[sel], K).astype(np.float64) * np.repeat(s[sel].astype(np.float64), group, 1) + \
        np.repeat(b[sel].astype(np.float64), group, 1)
    exact = x.astype(np.float64) @ W.T
    exact_r = x.astype(np.float64) @ bf(W).astype(np.float64).T      # with the weights as mx.dequantize returns them
    ys = []
    # up to 16 rows: the two tcgen05 forms (1: per-group products, scale applied after; 4: weights dequantised to bf16
    # first, accumulated in tensor memory) and the mma.sync form (0, the default; same arithmetic as 1)
    for form in (1, 4, 0):
        L.vk_w4_select(form)
        if force:
            L.vk_w4_force_plan(*force)
        try:
            y = ops.w4_gemm(tx, wt)
            y2 = ops.w4_gemm(tx, wt)
            ops.check_status()
        finally:
            L.vk_w4_force_plan(0, 0)
            L.vk_w4_select(0)
        assert torch.equal(y, y2), "the product must not depend on scheduling"
        got = y.float().cpu().numpy()
        np.testing.assert_allclose(got[:, sel], want, rtol=2e-2, atol=2e-2)
        # and much tighter against the exact product (forms 0 and 1 keep s*u + b unrounded, form 4 rounds it to bf16)
        # (beyond 16 rows only the last pass of up to 16 rows runs in the selected form: either product may be the nearer)
        err = np.abs(got[:, sel] - exact)
        if form == 4:
            err = np.minimum(err, np.abs(got[:, sel] - exact_r))
        assert (err <= 2.0 ** -8 * np.abs(exact) + 2e-3).all(), (form, err.max())
        ys.append(y)
    return ys[-1]


@pytest.mark.parametrize("M", [1, 2, 3, 4, 8, 9, 16])
def test_gemm_small(cuda, M):
    rng = np.random.default_rng(100 + M)
    _check_gemm(cuda, rng, M, 160, 512, 64)


@pytest.mark.parametrize("force", [(1, 0), (2, 0), (5, -1), (37, 1), (148, 0), (1000, 0), (0, -1), (0, 1)])
@pytest.mark.parametrize("group", [64, 128])
def test_gemm_plans(cuda, force, group):
    rng = np.random.default_rng(7)
    _check_gemm(cuda, rng, 16, 840, 1024, group, force=force)  # 4 superblocks of 256 rows, the last one ragged
    _check_gemm(cuda, rng, 5, 40, 1024, group, force=force)    # N not a multiple of 32


@pytest.mark.parametrize("N", [5120, 22016, 44032])
@pytest.mark.parametrize("M", [1, 2, 4, 8, 16])
def test_gemm_sweep_shapes(cuda, M, N):
    rng = np.random.default_rng(1)
    cols = np.sort(rng.choice(N, size=384, replace=False))
    _check_gemm(cuda, rng, M, N, 5120, 64, cols=cols)


def test_row_result_independent_of_batch(cuda):
    """A row's output is the same whether it is multiplied alone or inside a batch of 16."""
    from volundr_mlx_b200 import ops

    rng = np.random.default_rng(3)
    N, K = 640, 5120
    w, s, b = make_w4(rng, N, K, 64)
    wt = ops.w4_repack(*to_dev(w, s, b, cuda), 64)
    x = torch.from_numpy(bf(rng.normal(0, 1, size=(16, K)))).to(cuda).to(torch.bfloat16)
    y16 = ops.w4_gemm(x, wt)
    for m in (1, 4, 8):
        assert torch.equal(ops.w4_gemm(x[:m].contiguous(), wt), y16[:m])


@pytest.mark.parametrize("M,N,K", [(37, 96, 512), (17, 300, 1024), (32, 520, 2048), (33, 520, 2048), (64, 5120, 1024),
                                   (128, 840, 1024), (150, 264, 512)])
def test_rows_beyond_16(cuda, M, N, K):
    """More than 16 rows (verify windows, prefill chunks): passes of 64 / 32 / up to 16 rows, each streaming the weights
    once; same bars as the small-M product. Against 16-row passes only the split of K over CTAs differs (one CTA per
    SM instead of two), i.e. the association of the fp32 partial sums: equal up to a bf16 rounding step."""
    from volundr_mlx_b200 import ops

    rng = np.random.default_rng(5 + M)
    y = _check_gemm(cuda, rng, M, N, K, 64)
    # the same rows, 16 at a time
    rng = np.random.default_rng(5 + M)
    w, s, b = make_w4(rng, N, K, 64)
    x = bf(rng.normal(0, 1, size=(M, K)))
    wt = ops.w4_repack(*to_dev(w, s, b, cuda), 64)
    tx = torch.from_numpy(x).to(cuda).to(torch.bfloat16)
    y16 = torch.cat([ops.w4_gemm(tx[m0:m0 + 16].contiguous(), wt) for m0 in range(0, M, 16)])
    torch.testing.assert_close(y.float(), y16.float(), rtol=2 ** -7, atol=1e-3)


def test_rejects_bad_arguments(cuda):
    from volundr_mlx_b200 import _lib

    L = _lib.lib()
    assert L.vk_w4_gemm(None, None, 100, None, 64, 1, 64, 100, None, 0, None) == -1  # K not a multiple of 64
    assert L.vk_w4_repack(None, None, None, 32, 512, 32, None, None) == -1           # group 32 unsupported


@pytest.mark.parametrize("M", [1, 7, 16, 21])
@pytest.mark.parametrize("N,K", [(300, 256), (2050, 1024)])
def test_bf16_streaming_gemm(cuda, M, N, K):
    """The unquantised linears (lm_head): y = bf16(x . W^T) on the same streaming kernel. Floating point only, so the
    reference here is the fp32 product of the same bf16 inputs; rtol 2e-2 / atol 2e-2 as for every bf16 output."""
    from volundr_mlx_b200 import _lib, ops

    gen = torch.Generator(device=cuda)
    gen.manual_seed(N + M)
    W = (torch.randn((N, K), device=cuda, generator=gen) * 0.05).to(torch.bfloat16)
    x = torch.randn((M, K), device=cuda, generator=gen).to(torch.bfloat16)
    wt = ops.bf16_repack(W)
    L = _lib.lib()
    for ctas in (0, 1, 7):
        L.vk_w4_force_plan(ctas, 0)
        try:
            y = ops.bf16_gemm(x, wt)
        finally:
            L.vk_w4_force_plan(0, 0)
        want = x.float() @ W.float().T
        torch.testing.assert_close(y.float(), want, rtol=2e-2, atol=2e-2)
    ops.check_status()
