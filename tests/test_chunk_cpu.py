"""Host-side layout of a chunk's virtual rows (volundr_mlx_b200.chunk) without a GPU: which request and which token
every row stands for when the requests bring different numbers of tokens, and the scratch capacity classes."""
import torch

from volundr_mlx_b200 import chunk as CH


def test_virtual_rows_ragged_and_uniform():
    off, rows, tpos = CH.virtual_rows([1, 4, 2])
    assert off.tolist() == [0, 1, 5] and off.dtype == torch.int32
    assert rows.tolist() == [0, 1, 1, 1, 1, 2, 2]
    assert tpos.tolist() == [0, 0, 1, 2, 3, 0, 1]
    off, rows, tpos = CH.virtual_rows([3, 3])          # T tokens each: row b * T + t
    assert off.tolist() == [0, 3] and rows.tolist() == [0, 0, 0, 1, 1, 1] and tpos.tolist() == [0, 1, 2, 0, 1, 2]
    # every (request, token) pair appears exactly once, in request order
    lens = [5, 1, 1, 17, 2]
    off, rows, tpos = CH.virtual_rows(lens)
    pairs = list(zip(rows.tolist(), tpos.tolist()))
    assert pairs == [(b, t) for b, n in enumerate(lens) for t in range(n)]
    assert all(int(off[b]) == sum(lens[:b]) for b in range(len(lens)))


def test_scratch_capacity_classes():
    assert [CH.scratch_capacity(r) for r in (1, 16, 17, 128, 129, 2048, 2049)] == [16, 16, 32, 128, 256, 2048, 4096]
