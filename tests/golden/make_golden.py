"""Generate the golden fixtures of tests/golden/ from the reference's own NumPy fp64 model.

Run where the reference checkout is available:  python tests/golden/make_golden.py /path/to/reference
It imports volundr-mlx/tests/reference.py (numpy only) and writes:
  tiny_ref_logits.npz  Ref.forward logits of the tiny model (tests/tiny.py shapes) on dense parameters drawn by
                       volundr_mlx_b200.synth.make_params(tiny_args(), seed, quant=False) for two seeds / lengths
  ref_small.npz        engram_hash_seq rows, w4_pack_row words and sinkhorn outputs on seeded inputs
The tests regenerate the same parameters from the seed and compare the oracle (and the CUDA path) with these."""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))
from volundr_mlx_b200 import synth  # noqa: E402


def ref_params(p, a):
    """Our parameter dict -> the reference model's names / shapes (conv1d weight [C, K, 1])."""
    q = {}
    for k, v in p.items():
        if k.endswith("conv1d.weight"):
            v = np.asarray(v)[:, :, None]
        q[k] = np.asarray(v, dtype=np.float64)
    return q


def main(ref_root):
    sys.path.insert(0, str(Path(ref_root) / "volundr-mlx" / "tests"))
    import reference as R

    out = {}
    for seed, T in ((0, 44), (1, 60)):
        a = synth.tiny_args()
        p = synth.make_params(a, seed, quant=False, dtype_round=False)
        ids = np.random.default_rng(seed).integers(0, a.vocab_valid, size=T)
        logits = R.Ref(ref_params(p, a), a.to_dict()).forward(ids)
        out[f"ids_{seed}"] = ids
        out[f"logits_{seed}"] = logits
    np.savez_compressed(HERE / "tiny_ref_logits.npz", **out)

    rng = np.random.default_rng(1234)
    ids = [int(i) for i in rng.integers(0, 248320, size=257)] + [248045, 248046, 248069, 0, 1]
    small = {"engram_ids": np.array(ids)}
    for rows in (1 << 20, 1024):
        for n in (2, 3):
            small[f"engram_{rows}_{n}"] = np.array(R.engram_hash_seq(ids, n, rows))
    q = rng.integers(-8, 8, size=(6, 64))
    small["w4_q"] = q
    small["w4_words"] = np.stack([R.w4_pack_row(r) for r in q])
    logits = (rng.standard_normal((200, 16)) * 3)
    logits[:10] += np.eye(4).reshape(16) * 16
    small["sinkhorn_in"] = logits
    small["sinkhorn_out"] = R.sinkhorn(logits.reshape(-1, 4, 4), 10)
    np.savez_compressed(HERE / "ref_small.npz", **small)
    print("wrote", [f.name for f in HERE.glob("*.npz")])


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
