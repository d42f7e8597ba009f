"""bf16 rounding on NumPy arrays. A "bf16 tensor" in the oracle is a float32 array whose values are all exactly
representable in bf16; bf(x) makes one (round to nearest even), as every `.astype(bfloat16)` of the reference does
(volundr.py:24 and throughout)."""
import numpy as np


def bf(x):
    """Round float32/float64 values to bf16 (nearest even), returned as float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    nan = np.isnan(x)
    r = ((u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))) & np.uint32(0xFFFF0000)).view(np.float32)
    if nan.any():
        r = np.where(nan, np.float32(np.nan), r)
    return r


def is_bf(x) -> bool:
    x = np.ascontiguousarray(x, dtype=np.float32)
    return bool(np.all((x.view(np.uint32) & np.uint32(0xFFFF)) == 0))


def bf_bits(x):
    """uint16 bit patterns of a bf16-valued float32 array."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    return (x.view(np.uint32) >> np.uint32(16)).astype(np.uint16)


def from_bf_bits(b):
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def bf_from_f64_exact(r, err):
    """Round to bf16 the exact value r + err, where r is float64 and err the exact remainder of the float64
    operation that produced it (|err| far below one ulp of r). Differs from bf(r) only when r sits exactly on a
    bf16 tie and err pushes it off."""
    r = np.asarray(r, dtype=np.float64)
    lo = bf(r.astype(np.float32))  # candidate (float32 conversion of these short sums is exact, see callers)
    # detect ties: r exactly halfway between two neighbouring bf16 values
    f32 = r.astype(np.float32)
    exact32 = f32.astype(np.float64) == r
    u = f32.view(np.uint32)
    tie = exact32 & ((u & np.uint32(0xFFFF)) == np.uint32(0x8000))
    if not tie.any():
        return lo
    down = (u & np.uint32(0xFFFF0000)).view(np.float32)          # truncation toward zero in magnitude
    up = ((u & np.uint32(0xFFFF0000)) + np.uint32(0x10000)).view(np.float32)
    away = np.sign(err) == np.sign(r)                              # the remainder pushes the magnitude up
    fixed = np.where(away, up, down)
    return np.where(tie & (err != 0), fixed, lo).astype(np.float32)
