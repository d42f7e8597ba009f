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


def pages_open(pos, lens, table, free_list, free_top):
    """Pages for a chunk: row b is about to hold positions pos[b] .. pos[b] + lens[b] - 1; every position that starts a
    page pops one (rows in order, positions in order), exactly what lens[b] calls of step_begin would hand out row by
    row. `table` is updated in place; returns the new free_top."""
    top = int(free_top)
    for b in range(len(pos)):
        p0, p1 = int(pos[b]), int(pos[b]) + int(lens[b])
        pi = (p0 + PAGE - 1) // PAGE
        while pi * PAGE < p1:
            top -= 1
            table[b, pi] = free_list[top]
            pi += 1
    return top


def pages_release(items, reverse, table, free_list, free_top):
    """Pages back to the pool: for every (row, first, last) the table entries [first, last) that hold a page are
    pushed onto free_list in ascending order (descending with `reverse`) and set to -1. `table` and `free_list` are
    updated in place; returns the new free_top. (A verify pass that rejected drafts returns the pages those drafts
    opened, batch_spec.py:160-199 has no counterpart because the reference's rows own fixed rings; a row that leaves
    the batch, batch.py:416-431, returns all of its pages.)"""
    top = int(free_top)
    for b, a, z in items:
        idx = range(z - 1, a - 1, -1) if reverse else range(a, z)
        for pi in idx:
            if table[b, pi] < 0:
                continue
            free_list[top] = table[b, pi]
            top += 1
            table[b, pi] = -1
    return top
