"""Single kernels through the C ABI against the oracle on identical inputs: the integer / index work bit for bit
(far-block selection, step descriptors and page allocation, Engram rows), floating point within the stated bars."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import paging as OP
from oracle.model import Oracle
from oracle.numerics import bf

pytestmark = pytest.mark.gpu


def bf_t(x, dev):
    return torch.from_numpy(bf(x)).to(dev).to(torch.bfloat16)


@pytest.mark.parametrize("per_kv", [True, False])
def test_far_block_selection_bit_exact(cuda, per_kv):
    """Top-k block indices == the oracle's _block_scores + _topk_blocks (volundr.py:601-618) on ragged rows up to 2048
    blocks, including coarse scores with many ties (lower index wins, test_volundr.py:159-168)."""
    from volundr_mlx_b200 import _lib, ops
    from volundr_mlx_b200.batch import _Geom

    L = _lib.lib()
    rng = np.random.default_rng(3 + per_kv)
    g = _Geom()
    g.Hq, g.KVH, g.D = 10, 2, 128
    g.W, g.C, g.topk = (128, 64, 32) if per_kv else (64, 4, 48)
    g.IH, g.Di, g.NS = 4, 128, (g.KVH if per_kv else 1)
    g.far_tokens = int(per_kv)
    spp = 64 // g.C
    g.max_pages = 2048 if per_kv else 128
    g.n_pages = g.max_pages + 17
    B = 6
    nblk_max = g.max_pages * spp
    # context lengths log-uniform (1K..128K for the 64-token blocks)
    pos = np.exp(rng.uniform(np.log(1024), np.log(g.max_pages * 64 - 1), size=B)).astype(np.int32)
    pos[0] = g.max_pages * 64 - 1
    table = np.stack([rng.permutation(g.n_pages)[: g.max_pages] for _ in range(B)]).astype(np.int32)
    nh = g.Hq // g.KVH if per_kv else g.IH
    q = bf(rng.normal(size=(B, g.Hq if per_kv else g.IH, 128)))
    shape = (g.n_pages, g.KVH, spp, 128) if per_kv else (g.n_pages, spp, 128)
    keys = bf(rng.normal(size=shape))
    keys[: g.n_pages // 2] = bf(np.round(keys[: g.n_pages // 2] * 2) / 2)  # coarse half: ties
    sel = torch.full((B, g.NS, g.topk), -7, dtype=torch.int32, device=cuda)
    nsel = torch.zeros((B, g.NS), dtype=torch.int32, device=cuda)
    scratch = torch.empty(L.vk_bcsa_select_scratch_bytes(ctypes.byref(g), B, nblk_max), dtype=torch.uint8, device=cuda)
    tq, tk = bf_t(q, cuda), bf_t(keys, cuda)
    tpos, ttab = torch.from_numpy(pos).to(cuda), torch.from_numpy(table).to(cuda)
    rc = L.vk_bcsa_select(ctypes.byref(g), tq.data_ptr(), tk.data_ptr(), tpos.data_ptr(), ttab.data_ptr(), scratch.data_ptr(),
                          nblk_max, sel.data_ptr(), nsel.data_ptr(), B, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    ops.check_status()
    got, gn = sel.cpu().numpy(), nsel.cpu().numpy()
    orc = Oracle.__new__(Oracle)
    orc.exact = False
    for b in range(B):
        nv = max(0, (int(pos[b]) - g.W + 1) // g.C)
        for ns in range(g.NS):
            if nv <= g.topk:
                want = np.arange(nv)
            else:
                j = np.arange(nv)
                pages = table[b][j // spp]
                kk = keys[pages, ns, j % spp] if per_kv else keys[pages, j % spp]
                qq = q[b, ns * nh:(ns + 1) * nh] if per_kv else q[b]
                want = Oracle.topk_blocks(orc.block_scores(qq, kk), g.topk)
            assert gn[b, ns] == len(want)
            assert np.array_equal(got[b, ns, : len(want)], want), (b, ns)
            assert (got[b, ns, len(want):] == -1).all()


def test_step_descriptors_and_page_allocation_bit_exact(cuda):
    """vk_batch_step_begin == the CPU packer over several steps: same pages in the same order from the shuffled pool,
    same descriptors; gathering a row's pages gives back the contiguous layout."""
    from volundr_mlx_b200 import _lib

    L = _lib.lib()
    rng = np.random.default_rng(9)
    B, max_pages, n_pages, W, C, topk = 7, 16, 96, 128, 64, 3
    pos = np.array([0, 63, 64, 127, 128, 500, 701], np.int32)
    table = np.full((B, max_pages), -1, np.int32)
    free = rng.permutation(n_pages).astype(np.int32)
    top = n_pages
    for b in range(B):  # pages the rows already hold
        for i in range((pos[b] + 63) // 64):
            top -= 1
            table[b, i] = free[top]
    t_pos, t_tab = torch.from_numpy(pos.copy()).to(cuda), torch.from_numpy(table.copy()).to(cuda)
    t_free, t_top = torch.from_numpy(free).to(cuda), torch.tensor([top], dtype=torch.int32, device=cuda)
    t_desc = torch.zeros((B, 8), dtype=torch.int32, device=cuda)
    st = torch.cuda.current_stream().cuda_stream
    for step in range(70):
        assert L.vk_batch_step_begin(t_pos.data_ptr(), t_tab.data_ptr(), max_pages, t_free.data_ptr(), t_top.data_ptr(),
                                     t_desc.data_ptr(), B, W, C, topk, st) == 0
        assert L.vk_batch_step_end(t_pos.data_ptr(), None, B, st) == 0
        desc, top = OP.step_begin(pos, table, free, top, W, C, topk)
        pos += 1
        assert np.array_equal(t_desc.cpu().numpy(), desc), step
        assert int(t_top.item()) == top
        assert np.array_equal(t_tab.cpu().numpy(), table)
    assert np.array_equal(t_pos.cpu().numpy(), pos)
    pool = rng.integers(0, 1000, size=(n_pages, 2, 64, 4)).astype(np.float32)
    flat = OP.gather_row(pool, table[6], int(pos[6]))
    for t in (0, 63, 64, int(pos[6]) - 1):
        assert np.array_equal(flat[:, t], pool[table[6][t // 64], :, t % 64])


def test_engram_rows_bit_exact(cuda):
    """vk_embed's n-gram rows == the reference's hand values and the oracle's wrapping-uint32 hash with carried ids
    (test_volundr.py:53-65)."""
    from volundr_mlx_b200 import _lib

    L = _lib.lib()
    rng = np.random.default_rng(1234)
    B, D, V, rows = 3, 64, 248320, 1 << 20
    embed = torch.zeros((V, D), dtype=torch.bfloat16, device=cuda)
    w = torch.ones(D, dtype=torch.bfloat16, device=cuda)
    H = torch.zeros((B, 4, D), dtype=torch.bfloat16, device=cuda)
    hn = torch.zeros((B, D), dtype=torch.bfloat16, device=cuda)
    prev = torch.full((B, 2), -1, dtype=torch.int32, device=cuda)
    out = torch.zeros((B, 2), dtype=torch.int32, device=cuda)
    orders = (ctypes.c_int * 4)(2, 3, 0, 0)
    seqs = [[5, 7] + [int(i) for i in rng.integers(0, V, size=40)], [248045, 248046, 248069, 0, 1] + [0] * 37,
            [int(i) for i in rng.integers(0, V, size=42)]]
    hist = [[-1, -1] for _ in range(B)]
    st = torch.cuda.current_stream().cuda_stream
    for t in range(42):
        tok = torch.tensor([s[t] for s in seqs], dtype=torch.int32, device=cuda)
        assert L.vk_embed(tok.data_ptr(), embed.data_ptr(), w.data_ptr(), H.data_ptr(), hn.data_ptr(), prev.data_ptr(),
                          out.data_ptr(), orders, 2, rows, B, D, 1e-6, st) == 0
        got = out.cpu().numpy()
        for b in range(B):
            hist[b].append(seqs[b][t])
            assert got[b, 0] == Oracle.engram_row(hist[b], 2, rows)
            assert got[b, 1] == Oracle.engram_row(hist[b], 3, rows)
        if t == 0:
            assert got[0, 0] == 6
        if t == 1:
            assert got[0, 0] == (6 * 1000033 + 8) % rows
