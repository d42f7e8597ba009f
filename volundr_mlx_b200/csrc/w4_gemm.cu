// INT4 affine (group 64 / 128) weight GEMM for 1..16 activation rows: y[M,N] = x[M,K] . dequant(w)[N,K]^T.
//
// Replaces mx.quantized_matmul as called by every nn.QuantizedLinear of the reference (volundr.py:185-190, 377-386,
// 645-648) and the reference's small-M kernel qmm_nax_prepped (agens-mlx-bench/smallm/qmm_nax.py:28-139). Like that
// kernel it multiplies the raw 4-bit codes on the tensor cores and applies scale and bias per (row, group) to the
// fp32 group product: acc += s * (x_g . u_g) + b * sum(x_g).
//
// Memory layout. The reference layout (convert.py:7-14: u32 [N, K/8], nibble j of a word = element 8w + j, lowest
// first; bf16 scales / biases [N, K/G]) is repacked once at load time (vk_w4_repack) into a stream of 1152-byte
// chunks, one per (32 output rows, 64 input columns):
//   bytes    0..1023  codes  [stripe 2][lane 32][kstep 4] u32 : for lane (g = lane / 4, t = lane % 4), stripe s,
//                     kstep q the word holds the mma.m16n8k16 A fragment of rows r0 = 16 s + g, r1 = r0 + 8 and
//                     columns c = 16 q + 2 t: nibbles {0: (r0,c) 4: (r0,c+1) 1: (r1,c) 5: (r1,c+1) 2: (r0,c+8)
//                     6: (r0,c+9) 3: (r1,c+8) 7: (r1,c+9)}, so (w >> 4 i) & 0x000F000F | 0x43004300 is fragment
//                     register i as two bf16 values 128 + u.
//   bytes 1024..1151  [g 8][4] u32 = (scale | bias << 16) of rows g, g + 8, 16 + g, 24 + g.
// Chunks of one 32-row block are consecutive over K, so a warp streams its rows with 1-D TMA bulk copies into a
// private shared-memory ring; no byte of the weights is read twice and the packed size equals the algorithmic
// N*K/2 + N*(K/64)*4 bytes.
//
// Work split. grid = (ceil(N/32 / WARPS), S): each warp owns one 32-row block, each CTA one of S slabs of K. With
// S > 1 the fp32 partial sums go to a workspace [S][N32][16]; the CTA that arrives last at a grid column (an arrival
// counter per column, left at zero again) adds them in slab order, so the result does not depend on scheduling
// (the reference lists batch-variant matmuls as an open problem, NOTES_BATCHED_SERVE.md:256-258; here a row's
// result is the same for every M).
#include "common.cuh"

namespace {

constexpr int kChunkBytes = 1152;
#ifndef VK_STAGES
#define VK_STAGES 4
#endif
#ifndef VK_CH
#define VK_CH 1
#endif
constexpr int kStages = VK_STAGES;   // ring depth per warp
constexpr int kCH = VK_CH;       // chunks per stage
constexpr size_t kCounterBytes = 16384;  // split-K arrival counters at the head of the workspace (4096 grid columns)

struct W4Params {
    const uint8_t* wp;      // packed weights
    const __nv_bfloat16* x; // [M, ldx]
    __nv_bfloat16* y;       // [M, ldy]
    float* part;            // [S][NB*32][16] when S > 1
    int* counters;          // one per grid column; zero between launches
    int M, N, NB, G, S, ldx, ldy, ksmax;
};

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t w, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(w), "r"(mask), "r"(orv));  // (a & b) | c
    return r;
}

// one packed word -> the four A-fragment registers (bf16 pairs holding 128 + code)
__device__ __forceinline__ void unpack_codes(uint32_t w, uint32_t (&a)[4]) {
    a[0] = lop3_and_or(w, 0x000F000Fu, 0x43004300u);
    a[1] = lop3_and_or(w >> 4, 0x000F000Fu, 0x43004300u);
    a[2] = lop3_and_or(w >> 8, 0x000F000Fu, 0x43004300u);
    a[3] = lop3_and_or(w >> 12, 0x000F000Fu, 0x43004300u);
}

// mma with a zero accumulator input (first k-step of a group)
__device__ __forceinline__ void mma_bf16_z(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}

template <int MT, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, (MT == 2 ? 3 : 4)) w4_gemm_kernel(const W4Params p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int MR = MT * 8;                              // activation rows held (M padded)
    constexpr int kStageBytes = kCH * kChunkBytes;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int nb = blockIdx.x * WARPS + warp;
    const bool active = nb < p.NB;
    const int split = blockIdx.y;
    const int kg0 = (int)((long long)split * p.G / p.S), kg1 = (int)((long long)(split + 1) * p.G / p.S);
    const int ks = kg1 - kg0;
    const int nit = (ks + kCH - 1) / kCH;
    const int XS = p.ksmax * 64 + 8;                        // x slab row stride (bf16 elements); +8 keeps ldmatrix conflict-free

    uint8_t* ring = smem + (size_t)warp * kStages * kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)WARPS * kStages * kStageBytes) + warp * kStages;
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem + (size_t)WARPS * kStages * kStageBytes + WARPS * kStages * 8);
    float* sxs = reinterpret_cast<float*>(xs + (size_t)MR * XS);
    __shared__ int s_last;

    const uint8_t* src = p.wp + ((size_t)nb * p.G + kg0) * kChunkBytes;
    if (active && lane == 0) {
        for (int s = 0; s < kStages; s++) mbar_init(&bars[s], 1);
        mbar_fence_init();
        // the weights depend on no earlier kernel: start streaming before waiting for the producer of x
        for (int it = 0; it < kStages && it < nit; it++) {
            const int cnt = min(kCH, ks - it * kCH);
            mbar_expect_tx(&bars[it], cnt * kChunkBytes);
            tma_bulk_g2s(ring + it * kStageBytes, src + (size_t)it * kStageBytes, cnt * kChunkBytes, &bars[it]);
        }
    }
    pdl_launch_dependents();
    pdl_wait();

    // ---- stage the activation slab x[:, kg0*64 : kg1*64] (rows >= M are zero) and its per-group sums
    {
        const int vec_per_row = ks * 8;                     // 16-byte vectors per row
        for (int i = threadIdx.x; i < MR * vec_per_row; i += WARPS * 32) {
            const int r = i / vec_per_row, v = i - r * vec_per_row;
            uint4 val = make_uint4(0, 0, 0, 0);
            if (r < p.M) val = *reinterpret_cast<const uint4*>(p.x + (size_t)r * p.ldx + (size_t)kg0 * 64 + v * 8);
            *reinterpret_cast<uint4*>(xs + (size_t)r * XS + v * 8) = val;
        }
        __syncthreads();
        // one (group, row) sum per 4 lanes: 16 elements each, added in order, then a 2-step xor tree
        const int nsum = ks * MR;
        for (int i0 = 0; i0 < nsum; i0 += WARPS * 8) {
            const int i = i0 + (threadIdx.x >> 2);
            float s = 0.f;
            int kgl = 0, m = 0;
            if (i < nsum) {
                kgl = i / MR; m = i - kgl * MR;
                const uint4* row = reinterpret_cast<const uint4*>(xs + (size_t)m * XS + kgl * 64 + (threadIdx.x & 3) * 16);
                const uint4 a = row[0], b = row[1];
                s = bf_lo(a.x); s += bf_hi(a.x); s += bf_lo(a.y); s += bf_hi(a.y);
                s += bf_lo(a.z); s += bf_hi(a.z); s += bf_lo(a.w); s += bf_hi(a.w);
                s += bf_lo(b.x); s += bf_hi(b.x); s += bf_lo(b.y); s += bf_hi(b.y);
                s += bf_lo(b.z); s += bf_hi(b.z); s += bf_lo(b.w); s += bf_hi(b.w);
            }
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            // position so that thread t reads {m = 2t, 2t+1, 8+2t, 9+2t} as one vector
            if (i < nsum && (threadIdx.x & 3) == 0)
                sxs[kgl * MR + ((m & 7) >> 1) * (2 * MT) + (m >> 3) * 2 + (m & 1)] = s;
        }
        __syncthreads();
    }

    float acc[2][MT][4];
#pragma unroll
    for (int s = 0; s < 2; s++)
#pragma unroll
        for (int j = 0; j < MT; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[s][j][e] = 0.f;

    bool ok = true;
    if (active) {
        // ldmatrix row address of this lane inside the x slab (without the k offset)
        const int lm_mat = lane >> 3, lm_r = lane & 7;
        const int lm_row = (MT == 2 ? (lm_mat >> 1) * 8 : 0) + lm_r;
        const uint32_t xs_lane = smem_u32(xs + (size_t)lm_row * XS + (lm_mat & 1) * 8);
        for (int it = 0; it < nit && ok; it++) {
            const int st = it % kStages;
            ok = mbar_wait(&bars[st], (it / kStages) & 1);
            if (!ok) break;
            const int cnt = min(kCH, ks - it * kCH);
            for (int c = 0; c < cnt; c++) {
                const uint8_t* ch = ring + st * kStageBytes + c * kChunkBytes;
                const uint4 w0 = *reinterpret_cast<const uint4*>(ch + lane * 16);
                const uint4 w1 = *reinterpret_cast<const uint4*>(ch + 512 + lane * 16);
                const uint4 sb = *reinterpret_cast<const uint4*>(ch + 1024 + g * 16);
                const int kgl = it * kCH + c;
                float d[2][MT][4];
                const uint32_t wq0[4] = {w0.x, w0.y, w0.z, w0.w};
                const uint32_t wq1[4] = {w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    uint32_t b[2 * MT];
                    const uint32_t addr = xs_lane + (uint32_t)(kgl * 64 + q * 16) * 2;
                    if constexpr (MT == 2) {
                        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3])
                                     : "r"(addr));
                    } else {
                        asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(b[0]), "=r"(b[1]) : "r"(addr));
                    }
                    uint32_t a[4];
                    unpack_codes(wq0[q], a);
#pragma unroll
                    for (int j = 0; j < MT; j++) {
                        if (q == 0) mma_bf16_z(d[0][j], a, b[2 * j], b[2 * j + 1]);
                        else mma_bf16(d[0][j], a, b[2 * j], b[2 * j + 1]);
                    }
                    unpack_codes(wq1[q], a);
#pragma unroll
                    for (int j = 0; j < MT; j++) {
                        if (q == 0) mma_bf16_z(d[1][j], a, b[2 * j], b[2 * j + 1]);
                        else mma_bf16(d[1][j], a, b[2 * j], b[2 * j + 1]);
                    }
                }
                // group epilogue: acc += s * (D - 128 sum x) + b * sum x = s * D + (b - 128 s) * sum x
                float sx[MT][2];
                if constexpr (MT == 2) {
                    const float4 v = *reinterpret_cast<const float4*>(sxs + kgl * MR + t * 4);
                    sx[0][0] = v.x; sx[0][1] = v.y; sx[1][0] = v.z; sx[1][1] = v.w;
                } else {
                    const float2 v = *reinterpret_cast<const float2*>(sxs + kgl * MR + t * 2);
                    sx[0][0] = v.x; sx[0][1] = v.y;
                }
                const uint32_t sbw[4] = {sb.x, sb.y, sb.z, sb.w};
#pragma unroll
                for (int s = 0; s < 2; s++) {
                    const float s0 = bf_lo(sbw[2 * s]), c0 = fmaf(-128.f, s0, bf_hi(sbw[2 * s]));
                    const float s1 = bf_lo(sbw[2 * s + 1]), c1 = fmaf(-128.f, s1, bf_hi(sbw[2 * s + 1]));
#pragma unroll
                    for (int j = 0; j < MT; j++) {
                        acc[s][j][0] = fmaf(c0, sx[j][0], fmaf(s0, d[s][j][0], acc[s][j][0]));
                        acc[s][j][1] = fmaf(c0, sx[j][1], fmaf(s0, d[s][j][1], acc[s][j][1]));
                        acc[s][j][2] = fmaf(c1, sx[j][0], fmaf(s1, d[s][j][2], acc[s][j][2]));
                        acc[s][j][3] = fmaf(c1, sx[j][1], fmaf(s1, d[s][j][3], acc[s][j][3]));
                    }
                }
            }
            __syncwarp();
            if (lane == 0 && it + kStages < nit) {
                const int nx = it + kStages;
                const int ncnt = min(kCH, ks - nx * kCH);
                mbar_expect_tx(&bars[st], ncnt * kChunkBytes);
                tma_bulk_g2s(ring + st * kStageBytes, src + (size_t)nx * kStageBytes, ncnt * kChunkBytes, &bars[st]);
            }
        }
        if (!ok) {
            // a copy never landed: give the ones still in flight a (bounded) chance to land before the CTA's shared
            // memory is released; the output of this block is then left unwritten (status word set)
            for (int s = 0; s < kStages; s++) mbar_wait(&bars[s], 0);
        }
    }

    if (active && ok) {
#pragma unroll
        for (int s = 0; s < 2; s++) {
#pragma unroll
            for (int j = 0; j < MT; j++) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int n = nb * 32 + s * 16 + g + h * 8;
                    const int m = j * 8 + 2 * t;
                    const float v0 = acc[s][j][2 * h], v1 = acc[s][j][2 * h + 1];
                    if (p.S > 1) {
                        __stcg(reinterpret_cast<float2*>(p.part + ((size_t)split * p.NB * 32 + n) * 16 + m), make_float2(v0, v1));
                    } else if (n < p.N) {
                        if (m < p.M) p.y[(size_t)m * p.ldy + n] = f2bf(v0);
                        if (m + 1 < p.M) p.y[(size_t)(m + 1) * p.ldy + n] = f2bf(v1);
                    }
                }
            }
        }
    }
    if (p.S == 1) return;

    // ---- split-K: the CTA that arrives last at this column of the grid adds the S partial sums in slab order
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int old = atomicAdd(&p.counters[blockIdx.x], 1);
        s_last = (old == p.S - 1);
        if (s_last) p.counters[blockIdx.x] = 0;  // leave the counter ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int n_base = blockIdx.x * WARPS * 32;
    for (int i = threadIdx.x; i < WARPS * 32 * MR; i += WARPS * 32) {
        const int nl = i / MR, m = i - nl * MR;
        const int n = n_base + nl;
        if (n >= p.N || m >= p.M) continue;
        float s = 0.f;
        for (int k = 0; k < p.S; k++) s += __ldcg(p.part + ((size_t)k * p.NB * 32 + n) * 16 + m);
        p.y[(size_t)m * p.ldy + n] = f2bf(s);
    }
}

// ------------------------------------------------------------------------------------------------ repack / dequant
// reference layout -> packed chunks. One thread per packed u32 (codes) or per scale word.
__global__ void w4_repack_kernel(const uint32_t* __restrict__ w, const __nv_bfloat16* __restrict__ sc,
                                 const __nv_bfloat16* __restrict__ bi, int N, int K, int group, uint8_t* __restrict__ out,
                                 int NB, int G) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)NB * G * 288;  // u32 words per chunk
    if (idx >= total) return;
    const size_t chunk = idx / 288;
    const int wi = (int)(idx - chunk * 288);
    const int nb = (int)(chunk / G), kg = (int)(chunk - (size_t)nb * G);
    uint32_t* dst = reinterpret_cast<uint32_t*>(out + chunk * kChunkBytes) + wi;
    const int KW = K / 8;
    if (wi < 256) {
        const int s = wi >> 7, lane = (wi >> 2) & 31, q = wi & 3;
        const int g = lane >> 2, t = lane & 3;
        const int r0 = nb * 32 + s * 16 + g, r1 = r0 + 8;
        const int c = kg * 64 + q * 16 + 2 * t;
        auto code = [&](int r, int k) -> uint32_t {
            if (r >= N) return 0u;
            return (w[(size_t)r * KW + (k >> 3)] >> (4 * (k & 7))) & 0xFu;
        };
        uint32_t v = code(r0, c) | (code(r1, c) << 4) | (code(r0, c + 8) << 8) | (code(r1, c + 8) << 12) |
                     (code(r0, c + 1) << 16) | (code(r1, c + 1) << 20) | (code(r0, c + 9) << 24) | (code(r1, c + 9) << 28);
        *dst = v;
    } else {
        const int j = wi - 256;  // [g][4]
        const int g = j >> 2, e = j & 3;
        const int r = nb * 32 + (e >> 1) * 16 + g + (e & 1) * 8;
        uint32_t v = 0;
        if (r < N) {
            const int gi = (kg * 64) / group;
            const int GQ = K / group;
            const uint16_t s = *reinterpret_cast<const uint16_t*>(&sc[(size_t)r * GQ + gi]);
            const uint16_t b = *reinterpret_cast<const uint16_t*>(&bi[(size_t)r * GQ + gi]);
            v = (uint32_t)s | ((uint32_t)b << 16);
        }
        *dst = v;
    }
}

// W[n][k] = bf16(s * u + b): the exact sum rounded once (fma in bf16 rounds the exact result once).
__global__ void w4_dequant_kernel(const uint32_t* __restrict__ w, const __nv_bfloat16* __restrict__ sc,
                                  const __nv_bfloat16* __restrict__ bi, int N, int K, int group,
                                  __nv_bfloat16* __restrict__ out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // one packed word
    const int KW = K / 8;
    if (idx >= (size_t)N * KW) return;
    const int n = (int)(idx / KW), wi = (int)(idx - (size_t)n * KW);
    const uint32_t word = w[idx];
    const int gi = (wi * 8) / group;
    const __nv_bfloat16 s = sc[(size_t)n * (K / group) + gi], b = bi[(size_t)n * (K / group) + gi];
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const __nv_bfloat16 u0 = __ushort_as_bfloat16((unsigned short)(0x4300u | ((word >> (8 * j)) & 0xFu)));
        const __nv_bfloat16 u1 = __ushort_as_bfloat16((unsigned short)(0x4300u | ((word >> (8 * j + 4)) & 0xFu)));
        const __nv_bfloat16 k128 = __ushort_as_bfloat16((unsigned short)0x4300u);
        const __nv_bfloat16 r0 = __hfma(__hsub(u0, k128), s, b);   // 128 + u - 128 is exact
        const __nv_bfloat16 r1 = __hfma(__hsub(u1, k128), s, b);
        o[j] = (uint32_t)__bfloat16_as_ushort(r0) | ((uint32_t)__bfloat16_as_ushort(r1) << 16);
    }
    *reinterpret_cast<uint4*>(out + (size_t)n * K + (size_t)wi * 8) = make_uint4(o[0], o[1], o[2], o[3]);
}

struct W4Plan {
    int warps, S, ksmax, mt;
    size_t smem;
};

size_t w4_smem_bytes(int warps, int mt, int ksmax) {
    const int MR = mt * 8;
    return (size_t)warps * kStages * kCH * kChunkBytes + (size_t)warps * kStages * 8 +
           (size_t)MR * (ksmax * 64 + 8) * 2 + (size_t)ksmax * MR * 4;
}

int g_force_warps = 0, g_force_split = 0;

// Choose warps per CTA and the number of K slabs: fill 148 SMs in whole waves while keeping slabs long enough that
// the per-CTA activation slab and the partial sums stay small next to the weights streamed.
W4Plan w4_plan(int M, int N, int K) {
    const int NB = (N + 31) / 32, G = K / 64;
    const int mt = M <= 8 ? 1 : 2;
    W4Plan best = {};
    double best_cost = 1e300;
    for (int warps : {8, 4}) {
        if (g_force_warps && warps != g_force_warps) continue;
        const int nctas_n = (NB + warps - 1) / warps;
        for (int S = 1; S <= G && S <= 64; S++) {
            if (g_force_split && S != g_force_split) continue;
            const int ksmax = (G + S - 1) / S;
            if (ksmax < 2 && S > 1) break;
            const size_t smem = w4_smem_bytes(warps, mt, ksmax);
            if (smem > 200 * 1024) continue;
            int occ = (int)((220 * 1024) / (smem + 1024));
            occ = occ < 1 ? 1 : occ;
            const int occ_thr = 2048 / (warps * 32);
            occ = occ > occ_thr ? occ_thr : occ;
            const int occ_reg = mt == 2 ? 3 : 4;   // __launch_bounds__ of the kernel
            occ = occ > occ_reg ? occ_reg : occ;
            const long long ctas = (long long)nctas_n * S;
            const long long slots = 148LL * occ;
            const long long waves = (ctas + slots - 1) / slots;
            // bytes through one SM, plus a fixed cost per wave (ramp-up / drain) and the partial-sum traffic
            double cost = (double)waves * ((double)occ * ksmax * warps * kChunkBytes + 24e3);
            cost += (double)ksmax * mt * 8 * 128 * occ * waves * 0.5;  // activation slab re-read from L2
            if (S > 1) cost += 2.0 * S * NB * 32 * 16 * 4 / 148.0 + 6e3;
            if (cost < best_cost) {
                best_cost = cost;
                best = {warps, S, ksmax, mt, smem};
            }
        }
    }
    return best;
}

template <int MT, int WARPS>
cudaError_t launch_gemm(const W4Params& p, const W4Plan& plan, cudaStream_t stream) {
    static size_t configured = 0;
    auto kern = w4_gemm_kernel<MT, WARPS>;
    if (plan.smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        configured = 200 * 1024;
    }
    dim3 grid((p.NB + WARPS - 1) / WARPS, p.S);
    return vk_launch(kern, grid, dim3(WARPS * 32), plan.smem, stream, p);
}

}  // namespace

extern "C" {

size_t vk_w4_packed_bytes(int N, int K) { return (size_t)((N + 31) / 32) * (K / 64) * kChunkBytes; }

int vk_w4_repack(const void* w, const void* scales, const void* biases, int N, int K, int group, void* packed,
                 cudaStream_t stream) {
    if (N <= 0 || K <= 0 || K % 64 != 0 || (group != 64 && group != 128) || K % group != 0) return VK_EINVAL;
    const int NB = (N + 31) / 32, G = K / 64;
    const size_t total = (size_t)NB * G * 288;
    w4_repack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
        (const uint32_t*)w, (const __nv_bfloat16*)scales, (const __nv_bfloat16*)biases, N, K, group, (uint8_t*)packed, NB, G);
    return (int)cudaGetLastError();
}

int vk_w4_dequant(const void* w, const void* scales, const void* biases, int N, int K, int group, void* out,
                  cudaStream_t stream) {
    if (N <= 0 || K <= 0 || K % 8 != 0 || group <= 0 || group % 8 != 0 || K % group != 0) return VK_EINVAL;
    const size_t total = (size_t)N * (K / 8);
    w4_dequant_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
        (const uint32_t*)w, (const __nv_bfloat16*)scales, (const __nv_bfloat16*)biases, N, K, group, (__nv_bfloat16*)out);
    return (int)cudaGetLastError();
}

void vk_w4_force_plan(int warps, int split) {
    g_force_warps = warps;
    g_force_split = split;
}

size_t vk_w4_workspace_bytes(int M, int N, int K) {
    if (M > 16) M = 16;
    const W4Plan pl = w4_plan(M, N, K);
    return kCounterBytes + (pl.S > 1 ? (size_t)pl.S * ((N + 31) / 32) * 32 * 16 * 4 : 0);
}

int vk_w4_gemm(const void* packed, const void* x, int ldx, void* y, int ldy, int M, int N, int K, void* workspace,
               size_t workspace_bytes, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0 || K % 64 != 0 || ldx % 8 != 0 || ldx < K || ldy < N) return VK_EINVAL;
    if (((uintptr_t)x & 15) || ((uintptr_t)packed & 15)) return VK_EINVAL;
    // rows beyond 16 re-stream the weights once per 16 rows
    for (int m0 = 0; m0 < M; m0 += 16) {
        const int m = M - m0 < 16 ? M - m0 : 16;
        const W4Plan pl = w4_plan(m, N, K);
        W4Params p;
        p.wp = (const uint8_t*)packed;
        p.x = (const __nv_bfloat16*)x + (size_t)m0 * ldx;
        p.y = (__nv_bfloat16*)y + (size_t)m0 * ldy;
        p.counters = (int*)workspace;
        p.part = (float*)((uint8_t*)workspace + kCounterBytes);
        p.M = m; p.N = N; p.NB = (N + 31) / 32; p.G = K / 64; p.S = pl.S; p.ldx = ldx; p.ldy = ldy; p.ksmax = pl.ksmax;
        if (pl.S > 1 && (workspace == nullptr || workspace_bytes < kCounterBytes + (size_t)pl.S * p.NB * 32 * 16 * 4)) return VK_ENOSPC;
        cudaError_t e;
        if (pl.mt == 1) e = pl.warps == 8 ? launch_gemm<1, 8>(p, pl, stream) : launch_gemm<1, 4>(p, pl, stream);
        else e = pl.warps == 8 ? launch_gemm<2, 8>(p, pl, stream) : launch_gemm<2, 4>(p, pl, stream);
        if (e != cudaSuccess) return (int)e;
    }
    return VK_OK;
}

}  // extern "C"
