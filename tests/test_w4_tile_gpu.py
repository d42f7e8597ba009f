"""The tcgen05 tile GEMM (vk_w4_gemm_tile: many activation rows, accumulator in tensor memory) against the oracle:
rtol / atol 2e-2 against the W4 product, and much tighter against the exact product with the weights dequantised to
bf16 first (the kernel's own definition: bf16(s * u + b) rounded once, then fp32 accumulation)."""
import numpy as np
import pytest
import torch

from oracle import w4 as OW
from oracle.numerics import bf

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda", 0)


def make_w4(rng, N, K, group):
    codes = rng.integers(0, 16, size=(N, K), dtype=np.uint8)
    w = OW.pack_codes(codes)
    s = bf(np.abs(rng.normal(0, 0.02, size=(N, K // group))) / 8 + 1e-4)
    b = bf(rng.normal(0, 0.01, size=(N, K // group)))
    return w, s, b


@pytest.mark.parametrize("shape", [(0, 0), (256, 1), (256, 2), (64, 1), (64, 2)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 512), (37, 520, 1024), (200, 300, 2048), (256, 5120, 1024),
                                   (300, 768, 640)])
def test_tile_gemm(cuda, M, N, K, shape):
    """Every tile shape (weight rows per CTA 256 / 64, one or two tiles of activation rows per CTA) gives the same result,
    bit for bit: the accumulation order along K does not depend on it. (0, 0) = chosen from the shape: up to 128 rows that
    is the split-K kernel, whose fp32 partial sums over K ranges are added in a fixed order: the same result on every
    call, and within one bf16 step of the whole-K accumulation."""
    from volundr_mlx_b200 import _lib, ops

    _lib.check(_lib.lib().vk_w4_tile_force(*shape), "vk_w4_tile_force")
    rng = np.random.default_rng(M + N + K)
    w, s, b = make_w4(rng, N, K, 64)
    x = bf(rng.normal(0, 1, size=(M, K)))
    dev = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a)).to(cuda).to(dt)
    wt = ops.w4_repack(torch.from_numpy(w.view(np.int32)).to(cuda), dev(s, torch.bfloat16), dev(b, torch.bfloat16), 64)
    tx = dev(x, torch.bfloat16)
    y = ops.w4_gemm_tile(tx, wt)
    y2 = ops.w4_gemm_tile(tx, wt)
    _lib.check(_lib.lib().vk_w4_tile_force(256, 1), "vk_w4_tile_force")
    y3 = ops.w4_gemm_tile(tx, wt)
    _lib.check(_lib.lib().vk_w4_tile_force(0, 0), "vk_w4_tile_force")
    ops.check_status()
    assert torch.equal(y, y2)
    if shape != (0, 0) or M > 128:
        assert torch.equal(y, y3)
    else:
        d = (y.float() - y3.float()).abs()
        assert bool((d <= 2.0 ** -7 * y3.float().abs() + 1e-3).all()), float(d.max())
    got = y.float().cpu().numpy()
    np.testing.assert_allclose(got, OW.matmul(x, w, s, b, 64), rtol=2e-2, atol=2e-2)
    Wd = OW.dequant(w, s, b, 64).astype(np.float64)          # bf16-valued
    exact = x.astype(np.float64) @ Wd.T
    err = np.abs(got - exact)
    assert (err <= 2.0 ** -8 * np.abs(exact) + 1e-3).all(), err.max()


@pytest.mark.parametrize("N", [5120, 22016, 44032])
def test_tile_gemm_sweep_shapes_against_oracle(cuda, N):
    """The shapes of the W4A16 sweep (K = 5120, N in {5120, 22016, 44032}; codes uniform, scales |N(0, 0.02)| / 8, biases
    N(0, 0.01), activations N(0, 1), seed 1) at the row counts of a verify window and of prefill chunks, M in {64, 128,
    512}: rtol / atol 2e-2 against the oracle's W4 product and 2^-8 |exact| + 2e-3 against the exact product of the
    bf16-dequantised weights (the reference's own kernel bar is max relative error 3.7e-3, smallm/NOTES.md:104-105)."""
    from volundr_mlx_b200 import ops

    K = 5120
    rng = np.random.Generator(np.random.PCG64(1))
    w, s, b = make_w4(rng, N, K, 64)
    dev = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a)).to(cuda).to(dt)
    wt = ops.w4_repack(torch.from_numpy(w.view(np.int32)).to(cuda), dev(s, torch.bfloat16), dev(b, torch.bfloat16), 64)
    Wd = OW.dequant(w, s, b, 64)                              # bf16-valued float32: exact in float32
    for M in (64, 128, 512):
        x = bf(rng.normal(0, 1, size=(M, K)))
        got = ops.w4_gemm_tile(dev(x, torch.bfloat16), wt).float().cpu().numpy()
        ops.check_status()
        # columns sampled across the whole weight (every 256-row superblock contributes), all rows: the float64 product
        cols = np.unique(np.concatenate([np.arange(0, N, 97), np.arange(N - 300, N)]))
        exact = x.astype(np.float64) @ Wd[cols].astype(np.float64).T
        err = np.abs(got[:, cols] - exact)
        assert (err <= 2.0 ** -8 * np.abs(exact) + 2e-3).all(), (M, float(err.max()))
        np.testing.assert_allclose(got[:, cols], bf(exact.astype(np.float32)), rtol=2e-2, atol=2e-2)
        # ... and every column against a float32 product (exact weights, accumulation error ~1e-6)
        full = x @ Wd.T
        np.testing.assert_allclose(got, full, rtol=2e-2, atol=2e-2)
