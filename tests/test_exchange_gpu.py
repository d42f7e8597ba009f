"""The in-kernel tensor-parallel exchange on ONE GPU, without kernels that wait for one another: two regions stand for
two ranks. "Rank 1" runs first with a small wait limit: it pushes its partial rows (data and sequence numbers) into rank 0's region,
then its own wait for rank 0 runs out, which must surface as status 4 (the bounded-wait path; the device stays
usable). "Rank 0" runs afterwards, finds rank 1's rows in place and must produce exactly the plain kernel's result on
the bf16 sum of the two partial rows. The real two-process exchange is covered by tests/test_tp_gpu.py."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda", 0)


def _regions(L, peer, _lib, rows, D, calls):
    nbytes = L.vk_ar_region_bytes(2, rows, D)
    assert nbytes > 0
    bases = (ctypes.c_void_p * 8)()
    handle = ctypes.create_string_buffer(64)
    for r in range(2):
        p = ctypes.c_void_p()
        _lib.check(L.vk_ar_alloc(nbytes, ctypes.byref(p), handle), "vk_ar_alloc")
        bases[r] = p.value
    descs = []
    for r in range(2):
        d = peer.ArDesc()
        _lib.check(L.vk_ar_fill(ctypes.byref(d), 2, r, rows, D, calls, bases), "vk_ar_fill")
        descs.append(d)
    return bases, descs


def test_exchange_sum_and_bounded_wait(cuda):
    from volundr_mlx_b200 import _lib, ops, peer

    L = _lib.lib()
    B, D, rows = 5, 1024, 8
    bases, (d0, d1) = _regions(L, peer, _lib, rows, D, 4)
    d1.spin_limit = 2000
    g = torch.Generator(device="cpu").manual_seed(5)
    bf = dict(dtype=torch.bfloat16, device=cuda)
    x = torch.randn(B, D, generator=g).to(**bf)
    w = (torch.randn(D, generator=g) * 0.1).to(**bf)
    r0 = torch.randn(B, D, generator=g).to(**bf)
    r1 = torch.randn(B, D, generator=g).to(**bf)
    st = torch.cuda.current_stream().cuda_stream
    p = lambda t: t.data_ptr()

    def run(r, desc, call):
        h2, hn = torch.empty(B, D, **bf), torch.empty(B, D, **bf)
        rc = r.clone()
        _lib.check(L.vk_add_rmsnorm_ar(p(x), p(rc), p(w), p(h2), p(hn), None, B, D, 1e-6, 1,
                                       ctypes.byref(desc) if desc is not None else None, call, st), "vk_add_rmsnorm_ar")
        return h2, hn, rc

    try:
        for call in (0, 3):   # two calls of the "step": different slots
            run(r1, d1, call)                                   # rank 1 pushes, then gives up waiting
            with pytest.raises(RuntimeError, match="flag"):
                ops.check_status(cuda)
            h2, hn, summed = run(r0, d0, call)                  # rank 0 finds rank 1's rows
            ops.check_status(cuda)
            want_r = (r0.float() + r1.float()).to(torch.bfloat16)
            assert torch.equal(summed, want_r)
            h2_ref, hn_ref, _ = run(want_r, None, 0)
            assert torch.equal(h2, h2_ref) and torch.equal(hn, hn_ref)
        # a descriptor that does not fit the call is refused before any launch
        assert L.vk_add_rmsnorm_ar(p(x), p(r0), p(w), None, p(hn), None, B, D, 1e-6, 1, ctypes.byref(d0), 4, st) == -1
        assert L.vk_add_rmsnorm_ar(p(x), p(r0), p(w), None, p(hn), None, rows + 1, D, 1e-6, 1, ctypes.byref(d0), 0, st) == -1
    finally:
        torch.cuda.synchronize()
        for r in range(2):
            L.vk_ar_free(bases[r])
