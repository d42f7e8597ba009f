"""The in-kernel tensor-parallel exchange on ONE GPU, without kernels that wait for one another: `world` regions stand
for the ranks. Ranks world - 1 .. 1 run first, one after the other, with a small wait limit: each pushes its partial
rows (data and sequence numbers) into every other region, then its own wait for the ranks that have not run yet runs
out, which must surface as status 4 (the bounded-wait path; the device stays usable). "Rank 0" runs last, finds every
other rank's rows in place and must produce exactly the plain kernel's result on the bf16 of the fp32 sum, in rank
order, of the partial rows (two, six and eight ranks). The real two-process exchange is covered by tests/test_tp_gpu.py."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda", 0)


def _regions(L, peer, _lib, rows, D, calls, world=2):
    nbytes = L.vk_ar_region_bytes(world, rows, D)
    assert nbytes > 0
    bases = (ctypes.c_void_p * 8)()
    handle = ctypes.create_string_buffer(64)
    for r in range(world):
        p = ctypes.c_void_p()
        _lib.check(L.vk_ar_alloc(nbytes, ctypes.byref(p), handle), "vk_ar_alloc")
        bases[r] = p.value
    descs = []
    for r in range(world):
        d = peer.ArDesc()
        _lib.check(L.vk_ar_fill(ctypes.byref(d), world, r, rows, D, calls, bases), "vk_ar_fill")
        descs.append(d)
    return bases, descs


@pytest.mark.parametrize("world", [2, 6, 8])
def test_exchange_sum_and_bounded_wait(cuda, world):
    from volundr_mlx_b200 import _lib, ops, peer

    L = _lib.lib()
    B, D, rows = 5, 1024, 8
    bases, descs = _regions(L, peer, _lib, rows, D, 4, world)
    for d in descs[1:]:
        d.spin_limit = 2000
    g = torch.Generator(device="cpu").manual_seed(5)
    bf = dict(dtype=torch.bfloat16, device=cuda)
    x = torch.randn(B, D, generator=g).to(**bf)
    w = (torch.randn(D, generator=g) * 0.1).to(**bf)
    parts = [torch.randn(B, D, generator=g).to(**bf) for _ in range(world)]
    st = torch.cuda.current_stream().cuda_stream
    p = lambda t: t.data_ptr()
    d0 = descs[0]
    r0 = parts[0]

    def run(r, desc, call):
        h2, hn = torch.empty(B, D, **bf), torch.empty(B, D, **bf)
        rc = r.clone()
        _lib.check(L.vk_add_rmsnorm_ar(p(x), p(rc), p(w), p(h2), p(hn), None, B, D, 1e-6, 1,
                                       ctypes.byref(desc) if desc is not None else None, call, st), "vk_add_rmsnorm_ar")
        return h2, hn, rc

    try:
        for call in (0, 3):   # two calls of the "step": different slots
            for r in range(world - 1, 0, -1):                   # rank r pushes, then gives up waiting for the ranks below it
                run(parts[r], descs[r], call)
                with pytest.raises(RuntimeError, match="flag"):
                    ops.check_status(cuda)
            h2, hn, summed = run(r0, d0, call)                  # rank 0 finds everybody's rows
            ops.check_status(cuda)
            acc = torch.zeros(B, D, dtype=torch.float32, device=cuda)
            for r in range(world):
                acc = acc + parts[r].float()
            want_r = acc.to(torch.bfloat16)
            assert torch.equal(summed, want_r)
            h2_ref, hn_ref, _ = run(want_r, None, 0)
            assert torch.equal(h2, h2_ref) and torch.equal(hn, hn_ref)
        # a descriptor that does not fit the call is refused before any launch
        assert L.vk_add_rmsnorm_ar(p(x), p(r0), p(w), None, p(hn), None, B, D, 1e-6, 1, ctypes.byref(d0), 4, st) == -1
        assert L.vk_add_rmsnorm_ar(p(x), p(r0), p(w), None, p(hn), None, rows + 1, D, 1e-6, 1, ctypes.byref(d0), 0, st) == -1
    finally:
        torch.cuda.synchronize()
        for r in range(world):
            L.vk_ar_free(bases[r])
