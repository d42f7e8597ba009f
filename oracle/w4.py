"""INT4 affine weights: packing, dequantisation and the small-M product.

Layout (volundr-mlx/convert.py:7-14, :82-96; tests/reference.py:26-36 `w4_pack_row`): codes u in [0, 15] packed
eight to a uint32, nibble j of word w = element 8 w + j, lowest nibble first; bf16 scales and biases [N, K/G].
The reference converter always has bias = -8 scale (convert.py:11-14) and its test pins dequant == bf16(q * scale)
exactly for that case (tests/test_volundr.py:127-156). For a free bias the rounding of s*u + b inside
mx.dequantize is not pinned by any reference test ("parity unpinned"); it is defined here as the exact sum rounded
once to bf16, which agrees with the pinned case because s*(u-8) is exact in fp32."""
import numpy as np

from .numerics import bf, bf_from_f64_exact


def pack_codes(u):
    """u [N, K] ints in [0, 15] -> uint32 [N, K/8] (tests/reference.py:26-36 with nibble = q + 8 already applied)."""
    u = np.asarray(u, dtype=np.uint32)
    N, K = u.shape
    assert K % 8 == 0 and u.max() <= 15
    w = np.zeros((N, K // 8), dtype=np.uint32)
    for j in range(8):
        w |= u[:, j::8] << np.uint32(4 * j)
    return w


def unpack_codes(w, K):
    w = np.asarray(w, dtype=np.uint32)
    N = w.shape[0]
    u = np.zeros((N, K), dtype=np.uint32)
    for j in range(8):
        u[:, j::8] = (w >> np.uint32(4 * j)) & np.uint32(0xF)
    return u


def dequant(w, scales, biases, group, block_rows=4096):
    """bf16(s * u + b), the exact sum rounded once -> float32 [N, K] (bf16-valued). Large matrices go through in
    blocks of rows (the float64 temporaries of a 44032 x 5120 weight would otherwise take several GB)."""
    N = np.asarray(scales).shape[0]
    if N <= block_rows:
        return _dequant_block(w, scales, biases, group)
    out = np.empty((N, np.asarray(scales).shape[1] * group), dtype=np.float32)
    for r0 in range(0, N, block_rows):
        out[r0:r0 + block_rows] = _dequant_block(w[r0:r0 + block_rows], scales[r0:r0 + block_rows],
                                                 biases[r0:r0 + block_rows], group)
    return out


def _dequant_block(w, scales, biases, group):
    """s * u is exact in float64 (8-bit by 4-bit significands); the float64 sum's remainder is recovered with TwoSum."""
    s = np.asarray(scales, dtype=np.float64)
    b = np.asarray(biases, dtype=np.float64)
    N, Gq = s.shape
    K = Gq * group
    u = unpack_codes(w, K).astype(np.float64)
    p = u * np.repeat(s, group, axis=1)
    bb = np.repeat(b, group, axis=1)
    r = p + bb
    bv = r - p
    err = (p - (r - bv)) + (bb - bv)  # TwoSum remainder: p + bb == r + err exactly
    return bf_from_f64_exact(r, err)


def affine(w, scales, biases, group, dtype=np.float64, block_rows=4096):
    """s * u + b WITHOUT the rounding to bf16 -> [N, K] of `dtype`: the weight as a quantised matmul uses it.
    mx.quantized_matmul never materialises bf16 weights, and the reference's own small-M kernel forms, per group,
    s * (x_g . u_g) + b * sum(x_g) in fp32 (agens-mlx-bench/smallm/qmm_nax.py:56-67): algebraically x . (s u + b) with
    the unrounded weight. In float64 the value is exact (s * u has 12 significant bits, the sum with b fits easily); in
    float32 it is exact up to one rounding at 2^-24."""
    s = np.asarray(scales)
    N, Gq = s.shape
    K = Gq * group
    out = np.empty((N, K), dtype=dtype)
    for r0 in range(0, N, block_rows):
        u = unpack_codes(w[r0:r0 + block_rows], K).astype(np.float64)
        ss = np.repeat(np.asarray(scales[r0:r0 + block_rows], np.float64), group, axis=1)
        bb = np.repeat(np.asarray(biases[r0:r0 + block_rows], np.float64), group, axis=1)
        out[r0:r0 + block_rows] = u * ss + bb
    return out


def dequant_fast(w, scales, biases, group):
    """float32 s * u + b rounded to bf16, row block by row block: for timing the CPU baseline only (it can differ from
    `dequant` in the last bit where the float32 sum lands on a bf16 tie)."""
    s = np.asarray(scales, dtype=np.float32)
    b = np.asarray(biases, dtype=np.float32)
    N, Gq = s.shape
    K = Gq * group
    out = np.empty((N, K), dtype=np.float32)
    for r0 in range(0, N, 2048):
        u = unpack_codes(w[r0:r0 + 2048], K).astype(np.float32)
        out[r0:r0 + 2048] = bf(u * np.repeat(s[r0:r0 + 2048], group, axis=1) + np.repeat(b[r0:r0 + 2048], group, axis=1))
    return out


def matmul(x, w, scales, biases, group, acc=np.float64):
    """y = bf16(x . dequant(w)^T): what nn.QuantizedLinear computes (volundr.py:185-190), fp32 accumulation in the
    reference; float64 here so the oracle carries no accumulation-order noise of its own (tolerance rtol 2e-2)."""
    W = dequant(w, scales, biases, group).astype(acc)
    return bf((np.asarray(x, dtype=acc) @ W.T).astype(np.float32))
