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
    """Every tile shape (weight rows per CTA 256 / 64, one or two tiles of activation rows per CTA; (0, 0) = chosen
    from the shape) gives the same result, bit for bit: the accumulation order along K does not depend on it."""
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
    assert torch.equal(y, y2) and torch.equal(y, y3)
    got = y.float().cpu().numpy()
    np.testing.assert_allclose(got, OW.matmul(x, w, s, b, 64), rtol=2e-2, atol=2e-2)
    Wd = OW.dequant(w, s, b, 64).astype(np.float64)          # bf16-valued
    exact = x.astype(np.float64) @ Wd.T
    err = np.abs(got - exact)
    assert (err <= 2.0 ** -8 * np.abs(exact) + 1e-3).all(), err.max()
