"""CPU statement of the per-step row bookkeeping that the reference does on the host in BatchRows / BCSAStep
(volundr-mlx/batch.py:52-122), restated for a paged cache: page allocation from a free stack and the step
descriptor of every row. The reference has no page table (its rows live in per-row rings, batch.py:8-15), so the
packing itself is pinned by this statement, not by the reference; the index formulas are the reference's."""
import numpy as np

PAGE = 64


def step_begin(pos, table, free_list, free_top, W, C, topk):
    """Rows in order: a row whose next position opens a page pops one from free_list[--free_top]. Returns
    (desc [B, 8], new free_top); `table` is updated in place. desc = {pos, page, row in page, closes a block,
    nv = max(0, (p - W + 1) // C), nf = min(nv, topk), keys attended, window start} (batch.py:103-113)."""
    B = len(pos)
    desc = np.zeros((B, 8), np.int32)
    top = int(free_top)
    for b in range(B):
        p = int(pos[b])
        pi = p // PAGE
        if p % PAGE == 0:
            top -= 1
            table[b, pi] = free_list[top]
        nv = max(0, (p - W + 1) // C) if W > 0 else 0
        nf = min(nv, topk)
        lo = max(0, p - W + 1) if W > 0 else 0
        desc[b] = [p, table[b, pi], p % PAGE, int(W > 0 and (p + 1) % C == 0), nv, nf, (p - lo + 1) + nf, lo]
    return desc, top


def gather_row(pool, table_row, n_tokens):
    """pool [n_pages, KVH, PAGE, D] -> the row's contiguous [KVH, n_tokens, D] (the layout a ring-free B = 1 cache of
    the reference holds, volundr.py:443-460)."""
    npg = (n_tokens + PAGE - 1) // PAGE
    x = pool[table_row[:npg]]                       # [npg, KVH, PAGE, D]
    return np.transpose(x, (1, 0, 2, 3)).reshape(pool.shape[1], npg * PAGE, pool.shape[3])[:, :n_tokens]
