"""Batched speculative verify and per-row commit on the decode batch, with the reference's signatures
(batch_spec.verify_forward / commit, batch_spec.py:107-128, :173-199): every row of a BatchCache is fed its own T
tokens ([bonus, drafts]) at its own position in ONE pass over the weights, the caller reads the T logits rows per
request and decides how many tokens n_b each request keeps, and `commit` leaves every row exactly as if it had decoded
only its first n_b tokens.

Both are thin adapters over volundr_mlx_b200.chunk (forward_chunk(write=False) + commit_chunk), which holds the
arithmetic: B x T tokens as virtual rows, the tcgen05 tile GEMM from 64 rows on, vk_kda_chunk for the recurrence, the
chunk's K/V written to the pages and attended causally, and for the commit the KDA replay over the accepted prefix, the
open block's indexer keys, the Engram id window and the give-back of pages opened for rejected positions.
"""
from __future__ import annotations

from . import chunk as CH


def verify_forward(model, bc, ids, capture=()):
    """ids [B, T] int32 (tensor or nested lists): row b's [bonus, drafts] at its position. Returns (logits [B, T, vocab]
    bf16, features [B, T, len(capture) * hidden] of the capture layers or None, the commit record). The rows'
    positions do not move (commit does that). The record also carries the pass's greedy ids (`rec.greedy` [B, T] int32:
    first maximum over the valid vocabulary), which is what the acceptance rule of scheduler.py:462-465 compares the
    drafts with."""
    logits, _, rec = CH.forward_chunk(model, bc, ids, write=False, capture=tuple(capture))
    return logits, rec.features, rec


def commit(bc, rec, ns):
    """Row b keeps the first ns[b] (0..T; the reference always keeps at least the bonus token) of its T verified
    tokens; the rows' positions move by ns."""
    CH.commit_chunk(rec.model, bc, rec, ns)
