"""Batched verify and per-row commit on the decode cache (batch_spec.verify_forward / commit, batch_spec.py:107-199):
every row is fed T drafted tokens, the caller reads the T logits rows per request, decides how many drafts n_b each
request accepts, and `commit` leaves every row exactly as if it had decoded only its first n_b drafts.

This first form runs the T tokens as T steps of the decode path (one CUDA-graph replay each) and keeps what a rollback
needs: the state that cannot be recomputed (KDA state and conv window, the Engram id window) is copied after every step,
pages opened for rejected positions go back to the pool, and K/V (and pooled block means) written for rejected positions
are simply left behind: they lie beyond the row's position, are never read, and are overwritten when real tokens reach
them (a block is pooled again when it really closes). Logits and committed state are therefore those of sequential
decoding, bit for bit; what is not there yet is the speed of a verify tile that reads the weights once for all T
tokens.
"""
from __future__ import annotations

import torch

from . import batch as BT

PAGE = BT.PAGE


class Verify:
    """State between verify_forward and commit."""

    def __init__(self, bc, T):
        self.T = T
        self.pos0 = list(bc._pos)
        self.steps0 = bc.steps
        self.kda = [i for i, st in enumerate(bc.layers) if "S" in st]
        self.S = [[] for _ in self.kda]      # per KDA layer: state after 0..T tokens, rows [:B]
        self.conv = [[] for _ in self.kda]   # ... and the conv window
        self.engram = []
        self.free_top0 = None


def _snapshot(bc, v: Verify):
    B = bc.B
    par = bc._par()
    for j, i in enumerate(v.kda):
        st = bc.layers[i]
        v.S[j].append(st["S"][:B].clone())
        v.conv[j].append(st["conv"][par, :B].clone())
    v.engram.append(bc.engram_prev[:B].clone())


def verify_forward(model, bc, drafts):
    """drafts: [B][T] token ids (list of lists or int tensor), 1 <= T <= 16, the same T for every row. Returns
    (logits [B, T, V] bf16, greedy [B, T] int32, handle); logits[b, t] follow drafts[b][t]. The rows are left T tokens
    ahead: call commit(model, bc, handle, accepted) before anything else touches the cache."""
    d = torch.as_tensor(drafts, dtype=torch.int32)
    assert d.dim() == 2 and d.shape[0] == bc.B and 1 <= d.shape[1] <= 16
    B, T = d.shape
    for b in range(B):
        assert (bc._pos[b] + T + PAGE - 1) // PAGE <= bc.max_pages, "row would outgrow its page table"
    d = d.to(bc.pos.device)
    v = Verify(bc, T)
    _snapshot(bc, v)
    logits = torch.empty((B, T, bc.logits.shape[1]), dtype=bc.logits.dtype, device=bc.logits.device)
    greedy = torch.empty((B, T), dtype=torch.int32, device=bc.logits.device)
    for t in range(T):
        lg, _ = BT.forward(model, bc, d[:, t])
        logits[:, t] = lg
        greedy[:, t] = bc.greedy[:B]
        _snapshot(bc, v)
    return logits, greedy, v


def commit(model, bc, v: Verify, accepted):
    """accepted[b] in 0..T: the number of drafted tokens request b keeps (batch_spec.commit, batch_spec.py:160-199)."""
    B, T = bc.B, v.T
    acc = [int(x) for x in accepted]
    assert len(acc) == B and all(0 <= n <= T for n in acc)
    dev = bc.pos.device
    idx = torch.tensor(acc, dtype=torch.long, device=dev)
    rows = torch.arange(B, device=dev)
    par = bc._par()
    for j, i in enumerate(v.kda):
        st = bc.layers[i]
        st["S"][:B] = torch.stack(v.S[j])[idx, rows]
        st["conv"][par, :B] = torch.stack(v.conv[j])[idx, rows]
    bc.engram_prev[:B] = torch.stack(v.engram)[idx, rows]
    # pages opened at a rejected position go back to the pool (at most one per row: T <= 16 < 64)
    back = []
    for b in range(B):
        for t in range(acc[b], T):
            p = v.pos0[b] + t
            if p % PAGE == 0:
                back.append((b, p // PAGE))
    if back:
        torch.cuda.synchronize(dev)
        top = int(bc.free_top.item())
        for n, (b, pi) in enumerate(back):
            bc.free_list[top + n] = bc.table[b, pi]
            bc.table[b, pi] = -1
        bc.free_top += len(back)
    bc._pos = [v.pos0[b] + acc[b] for b in range(B)]
    bc.pos[:B] = torch.tensor(bc._pos, dtype=torch.int32, device=dev)
