// The activation layout the streaming GEMM reads ("x records"): per 64-column group one 2176-byte record,
//   bytes 0..2047    x[16 rows][64] bf16 as [piece 8][row 16][8 bf16]: the 16-byte piece c of row m (columns 8 c ..
//                    8 c + 7) sits at (c * 16 + m) * 16. The eight rows of a piece's 8 x 8 matrix are contiguous, which
//                    is what ldmatrix reads without bank conflicts and what a tcgen05 shared-memory operand without
//                    swizzle wants (core matrices of 8 rows x 16 bytes; 256 bytes between pieces along K, 128 bytes
//                    between the two row groups),
//   bytes 2048..2111 S[16 rows] fp32: the sum of the row's 64 values of this group (the values as stored, i.e. after
//                    their rounding to bf16), added in a fixed order; bytes 2112..2175 unused.
// Kernels that produce a GEMM input write their rows straight into records with these helpers (the reference fuses
// the same preparation into its producers: agens-mlx-bench/smallm/prep_nax.py:24-148). Rows a batch does not use
// must hold zeros.
#pragma once
#include "common.cuh"

constexpr int kXRecBytes = 2176;

// 16-byte piece `c` (0..7) of row m in group kg
__device__ __forceinline__ uint8_t* xrec_piece(uint8_t* xrec, int kg, int m, int c) {
    return xrec + (size_t)kg * kXRecBytes + ((c << 4) + m) * 16;
}
// element k (0..63) of row m in group kg
__device__ __forceinline__ __nv_bfloat16* xrec_elem(uint8_t* xrec, int kg, int m, int k) {
    return reinterpret_cast<__nv_bfloat16*>(xrec_piece(xrec, kg, m, k >> 3)) + (k & 7);
}
__device__ __forceinline__ void xrec_store_sum(uint8_t* xrec, int kg, int m, float s) {
    *reinterpret_cast<float*>(xrec + (size_t)kg * kXRecBytes + 2048 + m * 4) = s;
}
// Eight consecutive lanes hold the eight pieces of one (row, group): each lane's 8 values are added in order, then an
// xor tree over the lanes; the lane of piece 0 stores the sum words.
__device__ __forceinline__ void xrec_store_row_piece(uint8_t* xrec, int m, int piece_index, const float (&v)[8]) {
    const int kg = piece_index >> 3, c = piece_index & 7;
    uint4 u;
    u.x = pack_bf2(v[0], v[1]); u.y = pack_bf2(v[2], v[3]); u.z = pack_bf2(v[4], v[5]); u.w = pack_bf2(v[6], v[7]);
    *reinterpret_cast<uint4*>(xrec_piece(xrec, kg, m, c)) = u;
    float s = bf_lo(u.x); s += bf_hi(u.x); s += bf_lo(u.y); s += bf_hi(u.y);
    s += bf_lo(u.z); s += bf_hi(u.z); s += bf_lo(u.w); s += bf_hi(u.w);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    if (c == 0) xrec_store_sum(xrec, kg, m, s);
}
