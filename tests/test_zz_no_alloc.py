"""vk_bcsa_select_static: the far-block selection for callers that cannot allocate device memory (code that only
records launches into a CUDA graph, or a plugin living inside another runtime's memory pool, has no scratch buffer
to pass). It must return exactly what vk_bcsa_select returns with caller-provided scratch, call after call, although
every call reuses the same built-in array and finds the previous call's keys in it."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(dev, seed, per_kv):
    from volundr_mlx_b200.batch import _Geom

    rng = np.random.default_rng(seed)
    g = _Geom()
    g.Hq, g.KVH, g.D = 4, 2, 128
    g.W, g.C, g.topk = (128, 64, 5) if per_kv else (16, 4, 7)
    g.IH, g.Di, g.NS = 2, 128, (g.KVH if per_kv else 1)
    g.far_tokens = 1 if per_kv else 0
    g.max_pages, g.n_pages = 24, 200
    B = 6
    spp = 64 // g.C
    pos = rng.integers(0, g.max_pages * 64 - 1, size=B).astype(np.int32)
    pos[0] = 3                      # no far block
    pos[1] = g.W + g.C * g.topk     # exactly top-k valid blocks or fewer: the identity selection
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
