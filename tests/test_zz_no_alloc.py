"""vk_bcsa_select_static: the far-block selection for callers that cannot allocate device memory (code that only
records launches into a CUDA graph, or a plugin living inside another runtime's memory pool, has no scratch buffer
to pass). It must return exactly what vk_bcsa_select returns with caller-provided scratch, call after call, although
every call reuses the same built-in array and finds the previous call's keys in it."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(dev, seed, per_kv, max_pages=24, B=6, kvh=2, long_rows=False):
    from volundr_mlx_b200.batch import _Geom

    rng = np.random.default_rng(seed)
    g = _Geom()
    g.Hq, g.KVH, g.D = 2 * kvh, kvh, 128
    g.W, g.C, g.topk = (128, 64, 5) if per_kv else (16, 4, 7)
    g.IH, g.Di, g.NS = 2, 128, (g.KVH if per_kv else 1)
    g.far_tokens = 1 if per_kv else 0
    g.max_pages, g.n_pages = max_pages, max(200, max_pages + 40)
    spp = 64 // g.C
    pos = rng.integers(0, g.max_pages * 64 - 1, size=B).astype(np.int32)
    pos[0] = 3                      # no far block
    pos[1] = g.W + g.C * g.topk     # exactly top-k valid blocks or fewer: the identity selection
    if long_rows:                   # rows beyond the 512 blocks the kernel's shared-memory path holds: these use the array
        pos[2:] = rng.integers(g.W + 513 * g.C, g.max_pages * 64 - 1, size=B - 2)
        pos[-1] = g.max_pages * 64 - 1          # the row's last block: the highest index of its stretch of the array
    table = np.stack([rng.permutation(g.n_pages)[: g.max_pages] for _ in range(B)]).astype(np.int32)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    q = torch.randn((B, g.Hq if per_kv else g.IH, 128), device=dev, generator=gen).to(torch.bfloat16)
    # coarse values: many equal scores, so the tie rule (lower index wins) is exercised
    shape = (g.n_pages, g.KVH, spp, 128) if per_kv else (g.n_pages, spp, 128)
    keys = (torch.randint(-2, 3, shape, device=dev, generator=gen).float() * 0.25).to(torch.bfloat16)
    return g, B, torch.from_numpy(pos).to(dev), torch.from_numpy(table).to(dev), q, keys


def _both(L, g, B, pos, table, q, keys):
    dev = pos.device
    st = torch.cuda.current_stream().cuda_stream
    blocks = g.max_pages * (64 // g.C)
    out = []
    for static in (False, True):
        sel = torch.full((B, g.NS, g.topk), -7, dtype=torch.int32, device=dev)
        nsel = torch.full((B, g.NS), -7, dtype=torch.int32, device=dev)
        if static:
            rc = L.vk_bcsa_select_static(ctypes.byref(g), q.data_ptr(), keys.data_ptr(), pos.data_ptr(), table.data_ptr(),
                                         sel.data_ptr(), nsel.data_ptr(), B, st)
        else:
            scratch = torch.empty(L.vk_bcsa_select_scratch_bytes(ctypes.byref(g), B, blocks), dtype=torch.uint8, device=dev)
            rc = L.vk_bcsa_select(ctypes.byref(g), q.data_ptr(), keys.data_ptr(), pos.data_ptr(), table.data_ptr(),
                                  scratch.data_ptr(), blocks, sel.data_ptr(), nsel.data_ptr(), B, st)
        assert rc == 0, rc
        torch.cuda.synchronize()
        out.append((sel.cpu().numpy(), nsel.cpu().numpy()))
    return out


def test_static_scratch_selection_matches_and_repeats(cuda):
    from volundr_mlx_b200 import _lib, ops

    L = _lib.lib()
    # two calls in a row per mode, on different inputs: the second one finds the first one's keys in the array
    for seed, per_kv in ((1, True), (2, True), (3, False), (4, False)):
        g, B, pos, table, q, keys = _case(cuda, seed, per_kv)
        (sel_a, n_a), (sel_b, n_b) = _both(L, g, B, pos, table, q, keys)
        assert np.array_equal(n_a, n_b)
        assert np.array_equal(sel_a, sel_b)
        assert (n_a > 0).any() and (n_a == g.topk).any(), "the cases must reach the scoring path"
    ops.check_status()


def test_static_scratch_is_what_long_rows_sort_in(cuda):
    """Rows with more than 512 valid blocks do not fit the selection kernel's shared-memory path: their sort keys go
    through the scratch, here the built-in array. Two calls in a row per shape on different inputs (the second finds the
    first one's keys there), and the largest shape the entry point takes (16 rows x 8 groups x 2048 blocks), whose last
    row ends on the array's last element: a wrong address, stride or per-device look-up would show as wrong indices."""
    from volundr_mlx_b200 import _lib, ops

    L = _lib.lib()
    cases = [dict(per_kv=False, max_pages=128),                    # 2048 blocks of 4 positions, one shared group
             dict(per_kv=True, max_pages=1024),                    # 1024 blocks of 64 positions, a group per kv head
             dict(per_kv=True, max_pages=2048, B=16, kvh=8)]       # the capacity: B = 16, NS = 8, 2048 blocks
    for i, kw in enumerate(cases):
        for seed in (10 + 2 * i, 11 + 2 * i):
            g, B, pos, table, q, keys = _case(cuda, seed, long_rows=True, **kw)
            blocks = g.max_pages * (64 // g.C)
            nv = np.maximum(0, (pos.cpu().numpy() - g.W + 1) // g.C)
            assert (nv > 512).any() and nv.max() <= blocks and blocks <= 2048
            (sel_a, n_a), (sel_b, n_b) = _both(L, g, B, pos, table, q, keys)
            assert np.array_equal(n_a, n_b) and np.array_equal(sel_a, sel_b), kw
            assert (n_a == g.topk).any()
    ops.check_status()


def test_static_scratch_reports_a_position_beyond_the_page_table(cuda):
    """A position past max_pages * 64 is refused on the device by both entry points alike (status word, nothing
    selected), never used to index past the row's table."""
    from volundr_mlx_b200 import _lib, ops

    L = _lib.lib()
    g, B, pos, table, q, keys = _case(cuda, 20, True, max_pages=16)
    pos[2] = 16 * 64 + 64 * 700          # 700 blocks beyond the table's 16 (and beyond the shared-memory path)
    st = torch.cuda.current_stream().cuda_stream
    for static in (True, False):
        sel = torch.full((B, g.NS, g.topk), -7, dtype=torch.int32, device=cuda)
        nsel = torch.full((B, g.NS), -7, dtype=torch.int32, device=cuda)
        if static:
            rc = L.vk_bcsa_select_static(ctypes.byref(g), q.data_ptr(), keys.data_ptr(), pos.data_ptr(), table.data_ptr(),
                                         sel.data_ptr(), nsel.data_ptr(), B, st)
        else:
            scratch = torch.empty(L.vk_bcsa_select_scratch_bytes(ctypes.byref(g), B, 16), dtype=torch.uint8, device=cuda)
            rc = L.vk_bcsa_select(ctypes.byref(g), q.data_ptr(), keys.data_ptr(), pos.data_ptr(), table.data_ptr(),
                                  scratch.data_ptr(), 16, sel.data_ptr(), nsel.data_ptr(), B, st)
        assert rc == 0
        with pytest.raises(RuntimeError, match="index outside its pool"):
            ops.check_status()
        assert (nsel[2].cpu().numpy() == 0).all()


def test_static_scratch_rejects_what_does_not_fit(cuda):
    from volundr_mlx_b200 import _lib

    L = _lib.lib()
    g, B, pos, table, q, keys = _case(cuda, 5, True)
    g.max_pages = 4096          # 4096 blocks per row > 2048
    st = torch.cuda.current_stream().cuda_stream
    sel = torch.zeros((B, g.NS, g.topk), dtype=torch.int32, device=cuda)
    nsel = torch.zeros((B, g.NS), dtype=torch.int32, device=cuda)
    rc = L.vk_bcsa_select_static(ctypes.byref(g), q.data_ptr(), keys.data_ptr(), pos.data_ptr(), table.data_ptr(),
                                 sel.data_ptr(), nsel.data_ptr(), B, st)
    assert rc == -3
    g.max_pages = 24
    rc = L.vk_bcsa_select_static(ctypes.byref(g), q.data_ptr(), keys.data_ptr(), pos.data_ptr(), table.data_ptr(),
                                 sel.data_ptr(), nsel.data_ptr(), 17, st)   # 17 rows > 16
    assert rc == -3
