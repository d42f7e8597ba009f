"""CPU tests: the oracle against the fixtures generated from the reference's own NumPy fp64 model
(tests/golden/make_golden.py) and against the literal cases of the reference's tests."""
import numpy as np
import pytest

from oracle import w4 as OW
from oracle.model import Oracle, sinkhorn
from oracle.numerics import bf, bf_bits, is_bf
from volundr_mlx_b200 import synth
from pathlib import Path

GOLD = Path(__file__).resolve().parent / "golden"


def rel(a, b):
    return float(np.abs(np.asarray(a, np.float64) - b).max() / np.abs(b).max())


@pytest.mark.parametrize("seed", [0, 1])
def test_oracle_dataflow_matches_reference_fp64(seed):
    """Token-by-token decode through the oracle (no rounding) == the reference's whole-sequence fp64 model: KDA,
    Engram, BCSA with the far branch and top-k live, dense attention, mHC (test_volundr.py:270-285, bar 1e-4)."""
    g = np.load(GOLD / "tiny_ref_logits.npz")
    a = synth.tiny_args()
    p = synth.make_params(a, seed, quant=False, dtype_round=False)
    o = Oracle(a, p, exact=True)
    row = o.new_row()
    ids, ref = g[f"ids_{seed}"], g[f"logits_{seed}"]
    got = np.stack([o.step(row, int(t)) for t in ids])
    assert rel(got, ref) < 1e-9
    # the far branch is live: more valid blocks than top-k at the last position
    assert (len(ids) - 1 - a.bcsa_window + 1) // a.bcsa_compress > a.bcsa_topk


def test_oracle_bf16_close_to_fp64():
    """bf16 rounding points on: stays at the bf16 floor of the tiny model (test_volundr.py:301-317 accepts
    argmax agreement >= 90% and an error of the order of 1e-2 relative to the largest logit)."""
    g = np.load(GOLD / "tiny_ref_logits.npz")
    a = synth.tiny_args()
    p = synth.make_params(a, 1, quant=False)  # bf16-valued parameters
    ids = g["ids_1"]
    ex, lo = Oracle(a, p, exact=True), Oracle(a, p, exact=False)
    re, rl = ex.new_row(), lo.new_row()
    want = np.stack([ex.step(re, int(t)) for t in ids])
    got = np.stack([lo.step(rl, int(t)) for t in ids])
    assert is_bf(got)
    assert rel(got, want) < 5e-2
    v = a.vocab_valid
    assert (got[:, :v].argmax(-1) == want[:, :v].argmax(-1)).mean() >= 0.9


def test_engram_hash():
    """Hand values of the reference (test_volundr.py:53-65) and its u64 / 61-bit formula (tests/reference.py:12-23)."""
    rows = 1 << 20
    assert Oracle.engram_row([-1, 5], 2, rows) == 6
    assert Oracle.engram_row([5, 7], 2, rows) == (6 * 1000033 + 8) % rows
    g = np.load(GOLD / "ref_small.npz")
    ids = [-1, -1] + [int(i) for i in g["engram_ids"]]
    for r in (rows, 1024):
        for n in (2, 3):
            got = [Oracle.engram_row(ids[: t + 3], n, r) for t in range(len(ids) - 2)]
            assert np.array_equal(got, g[f"engram_{r}_{n}"]), (r, n)


def test_w4_pack_matches_reference_rows():
    """tests/reference.py:26-36: nibble = q + 8, lowest first."""
    g = np.load(GOLD / "ref_small.npz")
    words = OW.pack_codes(g["w4_q"] + 8)
    assert np.array_equal(words.view(np.int32), g["w4_words"])
    assert np.array_equal(OW.unpack_codes(words, 64), g["w4_q"] + 8)


def test_w4_dequant_pinned_case():
    """bias = -8 scale: dequant == bf16(q * scale) exactly (test_volundr.py:127-156), g64 and g128-stored-as-g64."""
    rng = np.random.default_rng(1234)
    n, k = 24, 512
    q = rng.integers(-8, 8, size=(n, k))
    for group, stored in ((128, 128), (128, 64), (64, 64)):
        s = bf(np.abs(rng.standard_normal((n, k // group))) * 0.01 + 1e-3)
        s_st = np.repeat(s, group // stored, axis=1)
        got = OW.dequant(OW.pack_codes(q + 8), s_st, bf(-8 * s_st), stored)
        assert np.array_equal(bf_bits(got), bf_bits(bf(q * np.repeat(s, group, axis=1))))
    x = bf(rng.standard_normal((5, k)))
    y = OW.matmul(x, OW.pack_codes(q + 8), s_st, bf(-8 * s_st), stored)
    assert rel(y, x.astype(np.float64) @ got.astype(np.float64).T) < 2e-2


def test_topk_tie_order():
    """The literal cases of test_volundr.py:159-168."""
    s = bf(np.array([1.0, 3.0, 3.0, 2.0, 3.0, -np.inf, 3.0, -1.0], np.float32))
    assert Oracle.topk_blocks(s, 3).tolist() == [1, 2, 4]
    s = bf(np.array([-1.0, -2.0, -0.5, -np.inf], np.float32))
    assert Oracle.topk_blocks(s, 1).tolist() == [2]
    rng = np.random.default_rng(1234)
    s = bf(rng.standard_normal((3, 700)))
    for r in s:
        ref = np.sort(np.argsort(-r, kind="stable")[:50])
        assert np.array_equal(Oracle.topk_blocks(r, 50), ref)


def test_sinkhorn():
    """vs the reference's fp64 sinkhorn incl. the identity-like regime, 2e-6 (test_volundr.py:68-75)."""
    g = np.load(GOLD / "ref_small.npz")
    got = sinkhorn(g["sinkhorn_in"].astype(np.float32).reshape(-1, 4, 4), 10, np.float32)
    assert np.abs(got - g["sinkhorn_out"]).max() < 2e-6


def test_library_exports_header_symbols():
    """Every function declared in include/volundr_b200.h is exported by the built library and bound by _lib."""
    import re
    from volundr_mlx_b200 import _lib, build

    build.build()
    hdr = (Path(__file__).resolve().parents[1] / "include" / "volundr_b200.h").read_text()
    names = set(re.findall(r"\b(vk_[a-z0-9_]+)\s*\(", hdr))
    L = _lib.lib()
    assert names, "no declarations found"
    for n in sorted(names):
        assert hasattr(L, n), n
        assert n in _lib.SIGNATURES, f"{n} is not bound in _lib.SIGNATURES"
    assert set(_lib.SIGNATURES) <= names, set(_lib.SIGNATURES) - names
