"""Tensor-parallel split of the model over the GPUs of one box: which rows / columns of every linear a rank holds.

The reference is single-GPU (no collective anywhere in it); this split is new design. Heads are the unit: attention
query / kv heads, KDA key / value heads with their state and KV pages stay on one rank; `gate_proj` / `up_proj` are
split by output column, `out_proj` / `o_proj` / `down_proj` by input column (row-parallel: partial sums are
all-reduced over the ranks), the lm_head by vocabulary rows. Pure index arithmetic (NumPy), shared by the GPU model
and by the CPU tests of the multi-rank logic."""
import numpy as np


def _block(r, per, cnt):
    """Rows of rank r when every rank owns `cnt` consecutive units of `per` rows."""
    return np.arange(r * cnt * per, (r + 1) * cnt * per)


def check(a, n):
    assert a.num_attention_heads % n == 0 and a.num_key_value_heads % n == 0, "attention heads must split evenly"
    assert a.linear_num_key_heads % n == 0 and a.linear_num_value_heads % n == 0, "KDA heads must split evenly"
    assert (a.linear_num_value_heads // n) % (a.linear_num_key_heads // n) == 0
    assert a.intermediate_size % (64 * n) == 0 and a.vocab_size % n == 0


def kda_rows(a, r, n):
    """Row indices of in_proj_qkv (q | k | v heads of this rank), in_proj_z, in_proj_b, f_up / dt_bias, and the input
    columns of out_proj."""
    K, V = a.linear_key_head_dim, a.linear_value_head_dim
    Hk, HV = a.linear_num_key_heads // n, a.linear_num_value_heads // n
    kd = a.linear_num_key_heads * K
    q = _block(r, K, Hk)
    qkv = np.concatenate([q, kd + q, 2 * kd + _block(r, V, HV)])
    return {"qkv": qkv, "z": _block(r, V, HV), "b": _block(r, 1, HV), "f_up": _block(r, K, HV),
            "out_cols": (r * HV * V, (r + 1) * HV * V)}


def attn_rows(a, r, n):
    D = a.head_dim
    Hq, KVH = a.num_attention_heads // n, a.num_key_value_heads // n
    return {"q": _block(r, 2 * D, Hq), "k": _block(r, D, KVH), "v": _block(r, D, KVH),
            "o_cols": (r * Hq * D, (r + 1) * Hq * D)}


def mlp_rows(a, r, n):
    I = a.intermediate_size // n
    return {"gate": _block(r, 1, I), "up": _block(r, 1, I), "down_cols": (r * I, (r + 1) * I)}


def vocab_rows(a, r, n):
    v = a.vocab_size // n
    return r * v, (r + 1) * v


def merge_argmax(vals, idxs):
    """Global greedy token from per-rank (max value, global index of its first maximum): the largest value wins, ties
    go to the lowest index (the first maximum of the full row, scheduler.py:391). vals, idxs: [ranks, B]."""
    vals, idxs = np.asarray(vals), np.asarray(idxs)
    out = np.zeros(vals.shape[1], dtype=np.int64)
    for b in range(vals.shape[1]):
        best = vals[:, b].max()
        out[b] = idxs[vals[:, b] == best, b].min()
    return out
