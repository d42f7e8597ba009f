// Fused row-wise kernels of the decode step: token embedding + first mHC norm, mHC mix (+ Sinkhorn) + input norm,
// residual add + post-attention norm, SiLU-gated product, mHC combine (+ Engram gate) + next norm, Engram row hashing
// and gather. One CTA per token row; every rounding to bf16 sits where the reference's ops path materialises a bf16
// array (volundr.py:264-290, 145-150, 166-168, 594-597; the fused reference kernels decode_fused.py:43-355 compute
// the same values).
#include "common.cuh"
#include "xrec.cuh"
#include "allreduce.cuh"
#include <cooperative_groups.h>

namespace {

constexpr int kEwThreads = 256;
constexpr int kEwWarps = kEwThreads / 32;

__device__ __forceinline__ float ldbf(const __nv_bfloat16* p, size_t i) { return bf2f(p[i]); }

// sum over the block in a fixed order (see block_sum)
__device__ __forceinline__ float ew_block_sum(float v, float* red) { return block_sum<kEwWarps>(v, red); }

// row kernels that move whole rows: one 16-byte piece (8 bf16) per thread and pass, blockDim = min(1024, D / 8 up to
// a warp multiple); sums over a block of any width in a fixed order
constexpr int kRowMaxWarps = 32;
__device__ __forceinline__ float row_block_sum(float v, float* red) {
    const int nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nw; i++) t += red[i];
    return t;
}
__device__ __forceinline__ void unpack8(const uint4 u, float (&x)[8]) {
    x[0] = bf_lo(u.x); x[1] = bf_hi(u.x); x[2] = bf_lo(u.y); x[3] = bf_hi(u.y);
    x[4] = bf_lo(u.z); x[5] = bf_hi(u.z); x[6] = bf_lo(u.w); x[7] = bf_hi(u.w);
}
__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&x)[8]) {
    unpack8(*reinterpret_cast<const uint4*>(p), x);
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&x)[8]) {
    uint4 u;
    u.x = pack_bf2(x[0], x[1]); u.y = pack_bf2(x[2], x[3]); u.z = pack_bf2(x[4], x[5]); u.w = pack_bf2(x[6], x[7]);
    *reinterpret_cast<uint4*>(p) = u;
}
static inline int row_threads(int D) {
    int t = ((D / 8 + 31) / 32) * 32;
    return t > 1024 ? 1024 : (t < 32 ? 32 : t);
}

// ------------------------------------------------------------------------------------------------ embedding
// x = embed[tok]; the four residual streams start as copies of x (volundr.py:929-930); hn = RMSNorm(x) * w0 is the
// first layer's mHC norm input (volundr.py:944). Also advances the Engram id window and hashes the n-gram rows
// (volundr.py:572-582, batch.py:526-529): row = (sum-product code over the last n ids, uint32 wrapping) & (rows - 1).
struct EmbedParams {
    const int* tok;                 // [B]
    const __nv_bfloat16* embed;     // [V, D]
    const __nv_bfloat16* w_mhc0;    // [D] plain RMSNorm weight of mhc[0]
    __nv_bfloat16* H;               // [B, 4, D]
    __nv_bfloat16* hn;              // [B, D]
    int* engram_prev;               // [B, keep] or null
    int* engram_rows_out;           // [B, n_orders]
    int D, keep, n_orders, engram_rows;
    int orders[4];
    float eps;
};

__global__ void __launch_bounds__(kEwThreads) embed_kernel(const EmbedParams p) {
    __shared__ float red[kEwWarps];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    const int tok = p.tok[b];
    const __nv_bfloat16* e = p.embed + (size_t)tok * p.D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < p.D; i += kEwThreads) {
        const __nv_bfloat16 v = e[i];
        const float f = bf2f(v);
        ss += f * f;
#pragma unroll
        for (int s = 0; s < 4; s++) p.H[((size_t)b * 4 + s) * p.D + i] = v;
    }
    ss = ew_block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)p.D + p.eps);
    for (int i = threadIdx.x; i < p.D; i += kEwThreads)
        p.hn[(size_t)b * p.D + i] = f2bf((bf2f(e[i]) * inv) * bf2f(p.w_mhc0[i]));
    if (p.engram_prev != nullptr && threadIdx.x == 0) {
        const uint32_t primes[5] = {1000003u, 1000033u, 1000037u, 1000039u, 1000081u};
        int full[8];
        for (int j = 0; j < p.keep; j++) full[j] = p.engram_prev[b * p.keep + j];
        full[p.keep] = tok;
        for (int o = 0; o < p.n_orders; o++) {
            const int n = p.orders[o];
            uint32_t code = 0;
            for (int j = 0; j < n; j++) code = code * primes[j % 5] + (uint32_t)(full[p.keep + 1 - n + j] + 1);
            p.engram_rows_out[b * p.n_orders + o] = (int)(code & (uint32_t)(p.engram_rows - 1));
        }
        for (int j = 0; j < p.keep; j++) p.engram_prev[b * p.keep + j] = full[j + 1];
    }
}

// ------------------------------------------------------------------------------------------------ mHC mix + norm
// ------------------------------------------------------------------------------------------------ mHC helpers
// The 24 dyn outputs of one row (bf16 linear D -> 24, volundr.py:302) by the whole CTA. Thread t holds the row's
// values hn[8 t .. 8 t + 7] (`on` = its piece exists). Order of the sum, the same wherever this is used: the thread's
// eight products as one fma chain, an xor tree over the warp, then the warps in order. part: [24][32] floats of shared
// memory; dsm[24] receives the bf16-rounded results (valid after the function's last barrier).
__device__ __forceinline__ void dyn24(const float (&hv)[8], bool on, int k, const __nv_bfloat16* __restrict__ w_dyn, int D,
                                      float* part, float* dsm, bool round_out = true) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int j0 = 0; j0 < 24; j0 += 8) {
        float acc[8];
        uint4 wv[8];
#pragma unroll
        for (int j = 0; j < 8; j++)
            wv[j] = on ? *reinterpret_cast<const uint4*>(w_dyn + (size_t)(j0 + j) * D + k) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float a = hv[0] * bf_lo(wv[j].x);
            a = fmaf(hv[1], bf_hi(wv[j].x), a);
            a = fmaf(hv[2], bf_lo(wv[j].y), a);
            a = fmaf(hv[3], bf_hi(wv[j].y), a);
            a = fmaf(hv[4], bf_lo(wv[j].z), a);
            a = fmaf(hv[5], bf_hi(wv[j].z), a);
            a = fmaf(hv[6], bf_lo(wv[j].w), a);
            a = fmaf(hv[7], bf_hi(wv[j].w), a);
            acc[j] = warp_sum(a);
        }
        if (lane == 0) {
#pragma unroll
            for (int j = 0; j < 8; j++) part[(j0 + j) * 32 + warp] = acc[j];
        }
    }
    __syncthreads();
    if (threadIdx.x < 24) {
        float a = 0.f;
        for (int w = 0; w < nw; w++) a += part[threadIdx.x * 32 + w];
        dsm[threadIdx.x] = round_out ? bfr(a) : a;   // (a cluster adds its CTAs' sums before rounding)
    }
    __syncthreads();
}

// res = bf(Sinkhorn_iters(exp(l - max))) of one row's 4 x 4 logits l = res_s + d[8:24], pre = bf(pre_s + d[0:4]),
// post = bf(post_s + d[4:8]) (volundr.py:264-271, :237-243). Called by all 32 lanes of one warp: lane i < 16 owns
// element (i / 4, i % 4); every row / column sum is formed in the order ((a0 + a1) + a2) + a3 from shuffled copies,
// the same additions a single thread would do.
// The static parts come in registers (mhc_static_load), so that their loads can be issued early.
struct MhcStatic { float res, pre, post; };   // lane i < 16: res_s[i]; lane < 4: pre_s[lane], post_s[lane]
__device__ __forceinline__ MhcStatic mhc_static_load(const __nv_bfloat16* __restrict__ pre_s, const __nv_bfloat16* __restrict__ post_s,
                                                     const __nv_bfloat16* __restrict__ res_s) {
    const int lane = threadIdx.x & 31;
    MhcStatic st;
    st.res = bf2f(res_s[lane & 15]);
    st.pre = bf2f(pre_s[lane & 3]);
    st.post = bf2f(post_s[lane & 3]);
    return st;
}
__device__ __forceinline__ void mhc_params_warp(const float* dsm, const MhcStatic st, int iters, float* pre_sm, float* post_out,
                                                float* res_out) {
    const int lane = threadIdx.x & 31;
    const int i = lane & 15, r = i >> 2, c = i & 3;
    const float l = st.res + dsm[8 + i];
    float mx = l;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float m = expf(l - mx);
    VK_TS(3, 9);
    for (int it = 0; it < iters; it++) {
        float a0 = __shfl_sync(0xffffffffu, m, 4 * r), a1 = __shfl_sync(0xffffffffu, m, 4 * r + 1);
        float a2 = __shfl_sync(0xffffffffu, m, 4 * r + 2), a3 = __shfl_sync(0xffffffffu, m, 4 * r + 3);
        m = m / fmaxf(((a0 + a1) + a2) + a3, 1e-9f);
        a0 = __shfl_sync(0xffffffffu, m, c); a1 = __shfl_sync(0xffffffffu, m, 4 + c);
        a2 = __shfl_sync(0xffffffffu, m, 8 + c); a3 = __shfl_sync(0xffffffffu, m, 12 + c);
        m = m / fmaxf(((a0 + a1) + a2) + a3, 1e-9f);
    }
    VK_TS(3, 10);
    if (lane < 16 && res_out != nullptr) res_out[i] = bfr(m);
    if (lane < 4) {
        pre_sm[lane] = bfr(st.pre + dsm[lane]);
        if (post_out != nullptr) post_out[lane] = bfr(st.post + dsm[4 + lane]);
    }
}

// d = dyn(hn) (bf16 linear D -> 24); pre = bf(pre_s + d[0:4]); post = bf(post_s + d[4:8]);
// res = bf(Sinkhorn_iters(exp(l - max))), l = res_s + d[8:24]; x_in = bf(((p0 + p1) + p2) + p3), p_s = bf(pre_s H_s);
// h = bf(x_in * rsqrt(mean x_in^2 + eps) * (1 + w_in)).   (volundr.py:319-322 with :264-278, :237-243, :132-150)
struct MixParams {
    const __nv_bfloat16* H;        // [B, 4, D]
    const __nv_bfloat16* hn;       // [B, D]
    const float* d;                // [B, 24] dyn(hn), bf16-valued
    const __nv_bfloat16* pre_s;    // [4]
    const __nv_bfloat16* post_s;   // [4]
    const __nv_bfloat16* res_s;    // [16]
    const __nv_bfloat16* w_in;     // [D] input_layernorm (offset norm)
    __nv_bfloat16* x_in;           // [B, D]
    __nv_bfloat16* h;              // [B, D]
    uint8_t* xrec_h;               // null, or D / 64 x records receiving h
    float* post;                   // [B, 4]  (bf16-valued)
    float* res;                    // [B, 16] (bf16-valued)
    int D, iters;
    float eps;
};

// d[b][j] = bf16(hn[b] . w_dyn[j]): one CTA of D / 8 threads per row (dyn24's order of summation). D <= 8192.
__global__ void __launch_bounds__(1024) mhc_dyn_kernel(const __nv_bfloat16* __restrict__ hn, const __nv_bfloat16* __restrict__ w_dyn,
                                                       float* __restrict__ d, int B, int D) {
    __shared__ float part[24 * 32];
    __shared__ float dsm[24];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x, k = threadIdx.x * 8;
    const bool on = k < D;
    float hv[8] = {};
    if (on) ld8(hn + (size_t)b * D + k, hv);
    dyn24(hv, on, k, w_dyn, D, part, dsm);
    if (threadIdx.x < 24) d[b * 24 + threadIdx.x] = dsm[threadIdx.x];
}

__global__ void __launch_bounds__(1024) mhc_mix_norm_kernel(const MixParams p) {
    __shared__ float red[kRowMaxWarps];
    __shared__ float pre_sm[4];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    const int D = p.D;
    if (threadIdx.x < 32)
        mhc_params_warp(p.d + b * 24, mhc_static_load(p.pre_s, p.post_s, p.res_s), p.iters, pre_sm, p.post + b * 4, p.res + b * 16);
    // (the other warps load their pieces of H meanwhile)
    const __nv_bfloat16* Hb = p.H + (size_t)b * 4 * D;
    const int k0 = threadIdx.x * 8;
    float h0[8], h1[8], h2[8], h3[8];
    if (k0 < D) { ld8(Hb + k0, h0); ld8(Hb + D + k0, h1); ld8(Hb + 2 * (size_t)D + k0, h2); ld8(Hb + 3 * (size_t)D + k0, h3); }
    __syncthreads();
    const float pr0 = pre_sm[0], pr1 = pre_sm[1], pr2 = pre_sm[2], pr3 = pre_sm[3];
    float ss = 0.f;
    float x0[8];
    for (int k = k0; k < D; k += blockDim.x * 8) {
        if (k != k0) { ld8(Hb + k, h0); ld8(Hb + D + k, h1); ld8(Hb + 2 * (size_t)D + k, h2); ld8(Hb + 3 * (size_t)D + k, h3); }
        float x[8];
#pragma unroll
        for (int e = 0; e < 8; e++) {
            x[e] = bfr(((bfr(pr0 * h0[e]) + bfr(pr1 * h1[e])) + bfr(pr2 * h2[e])) + bfr(pr3 * h3[e]));
            ss += x[e] * x[e];
        }
        st8(p.x_in + (size_t)b * D + k, x);
        if (k == k0) {
#pragma unroll
            for (int e = 0; e < 8; e++) x0[e] = x[e];
        }
    }
    ss = row_block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)D + p.eps);
    for (int k = k0; k < D; k += blockDim.x * 8) {
        float x[8], w[8], o[8];
        if (k == k0) {
#pragma unroll
            for (int e = 0; e < 8; e++) x[e] = x0[e];
        } else {
            ld8(p.x_in + (size_t)b * D + k, x);
        }
        ld8(p.w_in + k, w);
#pragma unroll
        for (int e = 0; e < 8; e++) o[e] = (x[e] * inv) * (1.f + w[e]);
        st8(p.h + (size_t)b * D + k, o);
        if (p.xrec_h != nullptr) xrec_store_row_piece(p.xrec_h, b, k >> 3, o);
    }
}

// ------------------------------------------------------------------------------------------------ add + norm
// h2 = bf(x + r); hn = bf(h2 * rsqrt(mean h2^2 + eps) * (off + w))      (volundr.py:893-899)
// Tensor-parallel: r holds this rank's partial product; the row's sum over ranks is formed first (allreduce.cuh).
__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x,
                                                           const __nv_bfloat16* r,
                                                           const __nv_bfloat16* __restrict__ w,
                                                           __nv_bfloat16* __restrict__ h2,
                                                           __nv_bfloat16* __restrict__ hn, uint8_t* __restrict__ xrec_hn,
                                                           int D, float eps, float offset, const VkArCall ar) {
    __shared__ float red[kRowMaxWarps];
    pdl_launch_dependents();   // (the dependent, a GEMM, reads only weights in front of its own wait)
    const int k0 = threadIdx.x * 8;
    const size_t base = (size_t)blockIdx.x * D;
    // in front of the wait: the weight, and x when r is given (x then comes from an earlier kernel than the one this
    // launch waits for, which produces r)
    float w0[8] = {}, x0[8] = {};
    if (k0 < D) {
        ld8(w + k0, w0);
        if (r != nullptr) ld8(x + base + k0, x0);
    }
    pdl_wait();
    if (r != nullptr) ar_reduce_row(ar, const_cast<__nv_bfloat16*>(r) + base, blockIdx.x, D);
    float ss = 0.f;
    float v0[8];
    for (int k = k0; k < D; k += blockDim.x * 8) {
        float v[8];
        if (k == k0 && r != nullptr) {
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = x0[e];
        } else {
            ld8(x + base + k, v);
        }
        if (r != nullptr) {
            float rv[8];
            ld8(r + base + k, rv);
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = bfr(v[e] + rv[e]);
        }
        if (h2 != nullptr) st8(h2 + base + k, v);
#pragma unroll
        for (int e = 0; e < 8; e++) ss += v[e] * v[e];
        if (k == k0) {
#pragma unroll
            for (int e = 0; e < 8; e++) v0[e] = v[e];
        }
    }
    ss = row_block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)D + eps);
    for (int k = k0; k < D; k += blockDim.x * 8) {
        float v[8], wv[8], o[8];
        if (k == k0) {
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = v0[e];
        } else {
            ld8(x + base + k, v);
            if (r != nullptr) {
                float rv[8];
                ld8(r + base + k, rv);
#pragma unroll
                for (int e = 0; e < 8; e++) v[e] = bfr(v[e] + rv[e]);
            }
        }
        if (k == k0) {
#pragma unroll
            for (int e = 0; e < 8; e++) wv[e] = w0[e];
        } else {
            ld8(w + k, wv);
        }
#pragma unroll
        for (int e = 0; e < 8; e++) o[e] = (v[e] * inv) * (offset + wv[e]);
        st8(hn + base + k, o);
        if (xrec_hn != nullptr) xrec_store_row_piece(xrec_hn, blockIdx.x, k >> 3, o);
    }
}

// ------------------------------------------------------------------------------------------------ silu(g) * u
// act = bf(silu(gate) * up) in fp32 (volundr.py:166-168); gu holds [gate (I) | up (I)] per row.
__global__ void __launch_bounds__(256) silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act,
                                                       uint8_t* __restrict__ xrec_act, int I, int ld_gu) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    const int piece = blockIdx.x * blockDim.x + threadIdx.x;   // 8 outputs
    const bool valid = piece * 8 < I;                           // (I is a multiple of 64: groups never straddle the edge)
    float g[8] = {}, u[8] = {}, o[8];
    if (valid) {
        ld8(gu + (size_t)b * ld_gu + piece * 8, g);
        ld8(gu + (size_t)b * ld_gu + I + piece * 8, u);
    }
#pragma unroll
    for (int e = 0; e < 8; e++) o[e] = (g[e] / (1.f + expf(-g[e]))) * u[e];
    if (valid && act != nullptr) st8(act + (size_t)b * I + piece * 8, o);
    if (xrec_act != nullptr) {   // whole warps take part in the group sums; pieces past the row write nothing
        if (valid) xrec_store_row_piece(xrec_act, b, piece, o);
        else { __shfl_xor_sync(0xffffffffu, 0.f, 1); __shfl_xor_sync(0xffffffffu, 0.f, 2); __shfl_xor_sync(0xffffffffu, 0.f, 4); }
    }
}

// ------------------------------------------------------------------------------------------------ Engram gather
// e = RMSNorm(concat_i table_i[row_i]) * w (volundr.py:594-595); table_i = columns [i dim, (i+1) dim) of one shared
// table when `shared`, else separate tables laid out one after another.
struct EngramGatherParams {
    const __nv_bfloat16* tables[4];
    const int* rows;               // [B, n_orders]
    const __nv_bfloat16* w;        // [n_orders * dim]
    __nv_bfloat16* e;              // [B, n_orders * dim]
    int n_orders, dim, ld_table[4], col0[4];
    float eps;
};

__global__ void __launch_bounds__(kEwThreads) engram_gather_kernel(const EngramGatherParams p) {
    __shared__ float red[kEwWarps];
    pdl_wait();
    pdl_launch_dependents();
    const int b = blockIdx.x;
    const int cat = p.n_orders * p.dim;
    float ss = 0.f;
    for (int i = threadIdx.x; i < cat; i += kEwThreads) {
        const int o = i / p.dim, c = i - o * p.dim;
        const int row = p.rows[b * p.n_orders + o];
        const float v = bf2f(p.tables[o][(size_t)row * p.ld_table[o] + p.col0[o] + c]);
        ss += v * v;
    }
    ss = ew_block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)cat + p.eps);
    for (int i = threadIdx.x; i < cat; i += kEwThreads) {
        const int o = i / p.dim, c = i - o * p.dim;
        const int row = p.rows[b * p.n_orders + o];
        const float v = bf2f(p.tables[o][(size_t)row * p.ld_table[o] + p.col0[o] + c]);
        p.e[(size_t)b * cat + i] = f2bf((v * inv) * bf2f(p.w[i]));
    }
}

// ------------------------------------------------------------------------------------------------ mHC combine + norm
// y = bf(h2 + m); Engram layers: y = bf(y + bf(g * val)), g = bf(sigmoid(bf(gate_w . y + gate_b))) (volundr.py:594-597);
// delta = bf(y - x_in); mixed_s = bf(sum_j res_sj H_j) (fp32, j in order); H'_s = bf(mixed_s + bf(post_s delta));
// mean = bf((((o0+o1)+o2)+o3) / 4)  (volundr.py:330-331, :281-290). Then either the next layer's mHC norm of the mean
// (plain RMSNorm, volundr.py:944-948) or, after the last layer, the model's final offset norm of stream 0 (:949).
struct CombineParams {
    __nv_bfloat16* H;              // [B, 4, D] in / out
    const __nv_bfloat16* h2;       // [B, D]
    const __nv_bfloat16* m;        // [B, D]
    const __nv_bfloat16* x_in;     // [B, D]
    const float* post;             // [B, 4]
    const float* res;              // [B, 16]
    const __nv_bfloat16* w_next;   // [D]
    __nv_bfloat16* hn;             // [B, D]
    const __nv_bfloat16* eng_val;  // [B, D] or null
    const __nv_bfloat16* eng_gate_w;  // [D]
    const __nv_bfloat16* eng_gate_b;  // [1]
    __nv_bfloat16* y_out;          // [B, D] or null (debug / tests)
    int D, final_norm;
    float eps;
    VkArCall ar;                   // tensor-parallel: m is this rank's partial product, summed over ranks first
};

__global__ void __launch_bounds__(1024) mhc_combine_norm_kernel(const CombineParams p) {
    __shared__ float red[kRowMaxWarps];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x, D = p.D;
    const size_t base = (size_t)b * D;
    ar_reduce_row(p.ar, const_cast<__nv_bfloat16*>(p.m) + base, b, D);
    const int k0 = threadIdx.x * 8;
    const int stride = blockDim.x * 8;
    float gate = 0.f;
    if (p.eng_val != nullptr) {
        float a = 0.f;
        for (int k = k0; k < D; k += stride) {
            float hv[8], mv[8], gw[8];
            ld8(p.h2 + base + k, hv); ld8(p.m + base + k, mv); ld8(p.eng_gate_w + k, gw);
#pragma unroll
            for (int e = 0; e < 8; e++) a = fmaf(bfr(hv[e] + mv[e]), gw[e], a);
        }
        a = row_block_sum(a, red);
        const float lin = bfr(a + bf2f(p.eng_gate_b[0]));
        gate = bfr(1.f / (1.f + expf(-lin)));
    }
    float r[16], po[4];
#pragma unroll
    for (int k = 0; k < 16; k++) r[k] = p.res[b * 16 + k];
#pragma unroll
    for (int s = 0; s < 4; s++) po[s] = p.post[b * 4 + s];
    __nv_bfloat16* Hb = p.H + (size_t)b * 4 * D;
    float ss = 0.f;
    float keep[8];
    for (int k = k0; k < D; k += stride) {
        float hv[8], mv[8], xv[8], hj[4][8], o[4][8], y[8], val[8];
        ld8(p.h2 + base + k, hv); ld8(p.m + base + k, mv); ld8(p.x_in + base + k, xv);
#pragma unroll
        for (int j = 0; j < 4; j++) ld8(Hb + (size_t)j * D + k, hj[j]);
        if (p.eng_val != nullptr) ld8(p.eng_val + base + k, val);
#pragma unroll
        for (int e = 0; e < 8; e++) {
            y[e] = bfr(hv[e] + mv[e]);
            if (p.eng_val != nullptr) y[e] = bfr(y[e] + bfr(gate * val[e]));
            const float delta = bfr(y[e] - xv[e]);
#pragma unroll
            for (int s = 0; s < 4; s++) {
                float mixed = r[4 * s] * hj[0][e];
                mixed = fmaf(r[4 * s + 1], hj[1][e], mixed);
                mixed = fmaf(r[4 * s + 2], hj[2][e], mixed);
                mixed = fmaf(r[4 * s + 3], hj[3][e], mixed);
                o[s][e] = bfr(bfr(mixed) + bfr(po[s] * delta));
            }
            const float v = p.final_norm ? o[0][e] : bfr((((o[0][e] + o[1][e]) + o[2][e]) + o[3][e]) * 0.25f);
            ss += v * v;
            if (k == k0) keep[e] = v;
        }
        if (p.y_out != nullptr) st8(p.y_out + base + k, y);
#pragma unroll
        for (int s = 0; s < 4; s++) st8(Hb + (size_t)s * D + k, o[s]);
    }
    if (p.w_next == nullptr) return;
    ss = row_block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)D + p.eps);
    const float off = p.final_norm ? 1.f : 0.f;
    for (int k = k0; k < D; k += stride) {
        float v[8], w[8], o[8];
        if (k == k0) {
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = keep[e];
        } else if (p.final_norm) {
            ld8(Hb + k, v);
        } else {
            float o0[8], o1[8], o2[8], o3[8];
            ld8(Hb + k, o0); ld8(Hb + (size_t)D + k, o1); ld8(Hb + 2 * (size_t)D + k, o2); ld8(Hb + 3 * (size_t)D + k, o3);
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = bfr((((o0[e] + o1[e]) + o2[e]) + o3[e]) * 0.25f);
        }
        ld8(p.w_next + k, w);
#pragma unroll
        for (int e = 0; e < 8; e++) o[e] = (v[e] * inv) * (off + w[e]);
        st8(p.hn + base + k, o);
    }
}

// ------------------------------------------------------------------------------------------------ layer boundary
// mhc_combine_norm of layer i followed by mhc_dyn + mhc_mix_norm of layer i + 1 in one kernel per row: the new streams
// stay in registers between the two halves, the mHC norm of their mean stays in registers for the 24 dyn dot
// products (all warps together), the 4 x 4 Sinkhorn runs on 16 lanes, and the next layer's input norm is written as a
// row and as x records. Same arithmetic, in the same order, as the three separate kernels (VolundrModel._fused_layers, volundr.py:945-948, runs them back to back).
struct BoundaryParams {
    CombineParams c;               // layer i (w_next = mhc[i + 1].norm; hn unused)
    const __nv_bfloat16* w_dyn;    // layer i + 1
    const __nv_bfloat16* pre_s;
    const __nv_bfloat16* post_s;
    const __nv_bfloat16* res_s;
    const __nv_bfloat16* w_in;
    __nv_bfloat16* x_in_out;       // [B, D] may alias c.x_in
    __nv_bfloat16* h;              // [B, D]
    uint8_t* xrec_h;
    float* post_out;               // [B, 4]  may alias c.post
    float* res_out;                // [B, 16] may alias c.res
    int iters;
};

constexpr int kBoundaryThreads = 640;

// CL = 1: one CTA of D / 8 threads per row. CL = 4: a cluster of four CTAs per row, each with a quarter of the row's
// 16-byte pieces; row-wide sums (norms, the engram gate, the 24 dyn products) are formed per CTA and then added over
// the cluster through distributed shared memory in rank order, the 4 x 4 Sinkhorn runs in every CTA (identical inputs,
// identical results) and rank 0 stores it. The row's arithmetic is spread over four SMs instead of one.
template <int CL>
__global__ void __launch_bounds__(kBoundaryThreads) mhc_boundary_kernel(const BoundaryParams q) {
    __shared__ float red[kRowMaxWarps];
    __shared__ float part[24 * 32];
    __shared__ float dsm[24];
    __shared__ float pre_sm[4];
    __shared__ float csum[4];      // this CTA's share of the row-wide sums: gate, ss, ss2 (read by the cluster)
    __shared__ float cdyn[24];     // ... and of the dyn products
    pdl_launch_dependents();   // (the dependent, a GEMM, reads only weights in front of its own wait)
    VK_TS(3, 0);
    const CombineParams& p = q.c;
    namespace cg = cooperative_groups;
    const int crank = CL > 1 ? (int)cg::this_cluster().block_rank() : 0;
    const int b = blockIdx.x / CL, D = p.D;
    const size_t base = (size_t)b * D;
    const int piece = crank * blockDim.x + threadIdx.x;
    const int k = piece * 8;
    const bool on = k < D;
    // sum over the row of a value every thread holds: block sum, then (CL > 1) the CTAs' sums in rank order
    auto row_sum = [&](float v, int slot) -> float {
        float t = row_block_sum(v, red);
        if constexpr (CL > 1) {
            cg::cluster_group cluster = cg::this_cluster();
            if (threadIdx.x == 0) csum[slot] = t;
            cluster.sync();
            t = 0.f;
#pragma unroll
            for (int r = 0; r < CL; r++) t += *cluster.map_shared_rank(&csum[slot], r);
        }
        return t;
    };
    // weights depend on no earlier kernel: fetch this thread's pieces, and start the 24 dyn rows towards L2, while the
    // kernel before this one is still running
    if (crank == 0 && threadIdx.x < 24) l2_prefetch_bulk(q.w_dyn + (size_t)threadIdx.x * D, (uint32_t)D * 2u);
    MhcStatic mst = {0.f, 0.f, 0.f};
    if (threadIdx.x < 32) mst = mhc_static_load(q.pre_s, q.post_s, q.res_s);
    uint4 w_next_raw = make_uint4(0u, 0u, 0u, 0u), w_in_raw = w_next_raw;
    if (on) {
        w_next_raw = *reinterpret_cast<const uint4*>(p.w_next + k);
        w_in_raw = *reinterpret_cast<const uint4*>(q.w_in + k);
    }
    // ... and so is everything this layer's earlier kernels and the previous boundary wrote (only m, and the Engram
    // value, come from the kernels right in front): the residual streams, x_in, h2, res / post
    float hv[8] = {}, mv[8] = {}, xv[8] = {};
    float r[16], po[4];
#pragma unroll
    for (int i = 0; i < 16; i++) r[i] = p.res[b * 16 + i];
#pragma unroll
    for (int s = 0; s < 4; s++) po[s] = p.post[b * 4 + s];
    __nv_bfloat16* Hb = p.H + (size_t)b * 4 * D;
    uint4 hraw[4] = {};
    if (on) {
        ld8(p.h2 + base + k, hv);
        ld8(p.x_in + base + k, xv);
#pragma unroll
        for (int j = 0; j < 4; j++) hraw[j] = *reinterpret_cast<const uint4*>(Hb + (size_t)j * D + k);
    }
    pdl_wait();
    VK_TS(3, 1);
    ar_reduce_span(p.ar, const_cast<__nv_bfloat16*>(p.m) + base, b, D, crank, CL);
    VK_TS(3, 2);
    float gate = 0.f;
    if (on) ld8(p.m + base + k, mv);
    float hj[4][8] = {};
    if (on) {
#pragma unroll
        for (int j = 0; j < 4; j++) unpack8(hraw[j], hj[j]);
    }
    if (p.eng_val != nullptr) {
        float a = 0.f;
        if (on) {
            float gw[8];
            ld8(p.eng_gate_w + k, gw);
#pragma unroll
            for (int e = 0; e < 8; e++) a = fmaf(bfr(hv[e] + mv[e]), gw[e], a);
        }
        a = row_sum(a, 0);
        gate = bfr(1.f / (1.f + expf(-bfr(a + bf2f(p.eng_gate_b[0])))));
    }
    float o[4][8] = {};
    float v[8] = {};
    float ss = 0.f;
    if (on) {
        float val[8];
        if (p.eng_val != nullptr) ld8(p.eng_val + base + k, val);
#pragma unroll
        for (int e = 0; e < 8; e++) {
            float y = bfr(hv[e] + mv[e]);
            if (p.eng_val != nullptr) y = bfr(y + bfr(gate * val[e]));
            const float delta = bfr(y - xv[e]);
#pragma unroll
            for (int s = 0; s < 4; s++) {
                float mixed = r[4 * s] * hj[0][e];
                mixed = fmaf(r[4 * s + 1], hj[1][e], mixed);
                mixed = fmaf(r[4 * s + 2], hj[2][e], mixed);
                mixed = fmaf(r[4 * s + 3], hj[3][e], mixed);
                o[s][e] = bfr(bfr(mixed) + bfr(po[s] * delta));
            }
            v[e] = bfr((((o[0][e] + o[1][e]) + o[2][e]) + o[3][e]) * 0.25f);
            ss += v[e] * v[e];
        }
#pragma unroll
        for (int s = 0; s < 4; s++) st8(Hb + (size_t)s * D + k, o[s]);
    }
    VK_TS(3, 3);
    ss = row_sum(ss, 1);
    VK_TS(3, 4);
    float hnv[8] = {};
    if (on) {
        const float inv = rsqrtf(ss / (float)D + p.eps);
        float w_next8[8];
        unpack8(w_next_raw, w_next8);
#pragma unroll
        for (int e = 0; e < 8; e++) hnv[e] = bfr((v[e] * inv) * w_next8[e]);   // the next layer's mHC norm, as bf16 values
    }
    // ---- dyn of the next layer from the norm just formed (registers), then its mHC parameters on warp 0
    if constexpr (CL > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        dyn24(hnv, on, k, q.w_dyn, D, part, cdyn, false);
        cluster.sync();
        if (threadIdx.x < 24) {
            float a = 0.f;
#pragma unroll
            for (int rk = 0; rk < CL; rk++) a += *cluster.map_shared_rank(&cdyn[threadIdx.x], rk);
            dsm[threadIdx.x] = bfr(a);
        }
        __syncthreads();
    } else {
        dyn24(hnv, on, k, q.w_dyn, D, part, dsm);
    }
    VK_TS(3, 5);
    if (threadIdx.x < 32)
        mhc_params_warp(dsm, mst, q.iters, pre_sm, crank == 0 ? q.post_out + b * 4 : nullptr,
                        crank == 0 ? q.res_out + b * 16 : nullptr);
    __syncthreads();
    VK_TS(3, 6);
    float x[8] = {};
    float ss2 = 0.f;
    if (on) {
#pragma unroll
        for (int e = 0; e < 8; e++) {
            x[e] = bfr(((bfr(pre_sm[0] * o[0][e]) + bfr(pre_sm[1] * o[1][e])) + bfr(pre_sm[2] * o[2][e])) + bfr(pre_sm[3] * o[3][e]));
            ss2 += x[e] * x[e];
        }
        st8(q.x_in_out + base + k, x);
    }
    ss2 = row_sum(ss2, 2);
    VK_TS(3, 7);
    const float inv2 = rsqrtf(ss2 / (float)D + p.eps);
    float ho[8] = {};
    if (on) {
        float w_in8[8];
        unpack8(w_in_raw, w_in8);
#pragma unroll
        for (int e = 0; e < 8; e++) ho[e] = (x[e] * inv2) * (1.f + w_in8[e]);
        st8(q.h + base + k, ho);
    }
    if (q.xrec_h != nullptr) {   // whole warps take part in the group sums
        if (on) xrec_store_row_piece(q.xrec_h, b, piece, ho);
        else { __shfl_xor_sync(0xffffffffu, 0.f, 1); __shfl_xor_sync(0xffffffffu, 0.f, 2); __shfl_xor_sync(0xffffffffu, 0.f, 4); }
    }
    if constexpr (CL > 1) cg::this_cluster().sync();   // nobody leaves while its shared memory may still be read
    VK_TS(3, 8);
}

// ------------------------------------------------------------------------------------------------ bf16 linear, few rows
// y[M, N] = bf16(x[M, K] . W[N, K]^T (+ bias)), fp32 accumulation: the linears the reference keeps unquantised
// (convert.py:16-17: lm_head, in_proj_b, mhc.dyn, BCSA indexer, Engram gate / value, f_up). One warp per output row.
template <int MMAX>
__global__ void __launch_bounds__(256) bf16_gemm_rows_kernel(const __nv_bfloat16* __restrict__ x, int ldx,
                                                            const __nv_bfloat16* __restrict__ W,
                                                            const __nv_bfloat16* __restrict__ bias,
                                                            __nv_bfloat16* __restrict__ y, int ldy, int M, int N, int K) {
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    if (n >= N) return;
    float acc[MMAX];
#pragma unroll
    for (int m = 0; m < MMAX; m++) acc[m] = 0.f;
    const __nv_bfloat16* wr = W + (size_t)n * K;
    for (int k = lane * 8; k < K; k += 256) {
        const uint4 wv = *reinterpret_cast<const uint4*>(wr + k);
        const float w0 = bf_lo(wv.x), w1 = bf_hi(wv.x), w2 = bf_lo(wv.y), w3 = bf_hi(wv.y);
        const float w4 = bf_lo(wv.z), w5 = bf_hi(wv.z), w6 = bf_lo(wv.w), w7 = bf_hi(wv.w);
#pragma unroll
        for (int m = 0; m < MMAX; m++) {
            if (m < M) {
                const uint4 xv = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + k);
                float a = acc[m];
                a = fmaf(bf_lo(xv.x), w0, a); a = fmaf(bf_hi(xv.x), w1, a);
                a = fmaf(bf_lo(xv.y), w2, a); a = fmaf(bf_hi(xv.y), w3, a);
                a = fmaf(bf_lo(xv.z), w4, a); a = fmaf(bf_hi(xv.z), w5, a);
                a = fmaf(bf_lo(xv.w), w6, a); a = fmaf(bf_hi(xv.w), w7, a);
                acc[m] = a;
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MMAX; m++) {
        if (m < M) {
            float t = warp_sum(acc[m]);
            if (lane == 0) {
                if (bias != nullptr) t += bf2f(bias[n]);
                y[(size_t)m * ldy + n] = f2bf(t);
            }
        }
    }
}

// The largest value of row[0 .. valid) and the lowest index that holds it, over a block of 1024 threads. The row is
// read in 16-byte pieces, four in flight per thread (a row of 150 thousand logits is 300 KB: one piece at a time per
// thread would pay the memory latency 19 times over); elements in front of the first 16-byte boundary and behind the
// last whole piece go one by one.
__device__ __forceinline__ void argmax_take(float v, int i, float& best, int& idx) {
    if (v > best || (v == best && i < idx)) { best = v; idx = i; }
}
__device__ __forceinline__ void argmax_row(const __nv_bfloat16* __restrict__ row, int valid, float& best, int& idx,
                                           float* bv, int* bi) {
    best = -INFINITY;
    idx = 0x7fffffff;
    int head = (int)(((16u - (unsigned)((uintptr_t)row & 15u)) & 15u) >> 1);
    head = head < valid ? head : valid;
    for (int i = threadIdx.x; i < head; i += blockDim.x) argmax_take(bf2f(row[i]), i, best, idx);
    const int nvec = (valid - head) >> 3;
    const uint4* v = reinterpret_cast<const uint4*>(row + head);
    const uint4 lowest = make_uint4(0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u);   // eight times -inf
    for (int j0 = threadIdx.x; j0 < nvec; j0 += 4 * blockDim.x) {
        uint4 x[4];
#pragma unroll
        for (int u = 0; u < 4; u++) x[u] = j0 + u * (int)blockDim.x < nvec ? v[j0 + u * (int)blockDim.x] : lowest;
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i0 = head + 8 * (j0 + u * (int)blockDim.x);
            const uint32_t w[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                argmax_take(bf_lo(w[e]), i0 + 2 * e, best, idx);
                argmax_take(bf_hi(w[e]), i0 + 2 * e + 1, best, idx);
            }
        }
    }
    for (int i = head + 8 * nvec + threadIdx.x; i < valid; i += blockDim.x) argmax_take(bf2f(row[i]), i, best, idx);
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        argmax_take(ov, oi, best, idx);
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0)
        for (int w = 1; w < (int)(blockDim.x >> 5); w++) argmax_take(bv[w], bi[w], best, idx);
}

// first maximum over logits[:, :vocab_valid] (scheduler.py:391)
__global__ void __launch_bounds__(1024) argmax_kernel(const __nv_bfloat16* __restrict__ logits, int ld, int valid,
                                                      int* __restrict__ out) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    float best;
    int idx;
    argmax_row(logits + (size_t)b * ld, valid, best, idx, bv, bi);
    if (threadIdx.x == 0) out[b] = idx;
}

// Vocabulary-sharded greedy token. Each rank: (bits of its largest valid logit, global index of its first maximum).
__global__ void __launch_bounds__(1024) argmax_pairs_kernel(const __nv_bfloat16* __restrict__ logits, int ld, int valid,
                                                            int index_offset, int* __restrict__ pairs) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    float best;
    int idx;
    argmax_row(logits + (size_t)b * ld, valid, best, idx, bv, bi);
    if (threadIdx.x == 0) {
        pairs[2 * b] = __float_as_int(best);
        pairs[2 * b + 1] = idx == 0x7fffffff ? idx : idx + index_offset;
    }
}

// pairs [ranks, B, 2] -> the largest value, ties to the lowest global index
__global__ void argmax_merge_kernel(const int* __restrict__ pairs, int n_ranks, int* __restrict__ out, int B) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int r = 0; r < n_ranks; r++) {
        const float v = __int_as_float(pairs[((size_t)r * B + b) * 2]);
        const int i = pairs[((size_t)r * B + b) * 2 + 1];
        if (v > best || (v == best && i < idx)) { best = v; idx = i; }
    }
    out[b] = idx;
}

}  // namespace

bool g_boundary_cluster = false;   // measured: no faster than one CTA per row (the kernel is bound by the latency of one
                                   // thread's chain of loads and roundings, not by the SM's issue rate); kept selectable

extern "C" {

// 1: vk_mhc_boundary spreads a row over a cluster of four CTAs when the hidden size allows; 0 (default): one CTA per row
void vk_mhc_boundary_set_cluster(int on) { g_boundary_cluster = on != 0; }

int vk_argmax_pairs(const void* logits, int ld, int valid, int index_offset, int* pairs, int B, cudaStream_t stream) {
    if (B <= 0) return VK_EINVAL;
    return (int)vk_launch(argmax_pairs_kernel, dim3(B), dim3(1024), 0, stream, (const __nv_bfloat16*)logits, ld,
                          valid < 0 ? 0 : valid, index_offset, pairs);
}

int vk_argmax_merge(const int* pairs, int n_ranks, int* out, int B, cudaStream_t stream) {
    if (B <= 0 || n_ranks <= 0) return VK_EINVAL;
    return (int)vk_launch(argmax_merge_kernel, dim3((B + 63) / 64), dim3(64), 0, stream, pairs, n_ranks, out, B);
}

int vk_embed(const int* tok, const void* embed, const void* w_mhc0, void* H, void* hn, int* engram_prev,
             int* engram_rows_out, const int* orders, int n_orders, int engram_rows, int B, int D, float eps,
             cudaStream_t stream) {
    if (B <= 0 || D <= 0 || n_orders < 0 || n_orders > 4) return VK_EINVAL;
    EmbedParams p = {};
    p.tok = tok; p.embed = (const __nv_bfloat16*)embed; p.w_mhc0 = (const __nv_bfloat16*)w_mhc0;
    p.H = (__nv_bfloat16*)H; p.hn = (__nv_bfloat16*)hn; p.engram_prev = engram_prev; p.engram_rows_out = engram_rows_out;
    p.D = D; p.n_orders = n_orders; p.engram_rows = engram_rows; p.eps = eps;
    int keep = 0;
    for (int i = 0; i < n_orders; i++) {
        if (orders[i] < 1 || orders[i] > 8) return VK_EINVAL;
        p.orders[i] = orders[i];
        keep = orders[i] - 1 > keep ? orders[i] - 1 : keep;
    }
    p.keep = keep;
    return (int)vk_launch(embed_kernel, dim3(B), dim3(kEwThreads), 0, stream, p);
}

int vk_mhc_mix_norm(const void* H, const void* hn, const void* w_dyn, const void* pre_s, const void* post_s,
                    const void* res_s, const void* w_in, void* x_in, void* h, void* xrec_h, float* post, float* res,
                    float* d_scratch, int B, int D, int iters, float eps, cudaStream_t stream) {
    if (B <= 0 || D <= 0 || D % 8 != 0 || d_scratch == nullptr || (xrec_h != nullptr && (D % 64 != 0 || B > 16))) return VK_EINVAL;
    if (D > 8192) return VK_ETOOBIG;
    VK_CUDA(vk_launch(mhc_dyn_kernel, dim3(B), dim3(row_threads(D)), 0, stream, (const __nv_bfloat16*)hn,
                      (const __nv_bfloat16*)w_dyn, d_scratch, B, D));
    MixParams p = {(const __nv_bfloat16*)H, (const __nv_bfloat16*)hn, d_scratch,
                   (const __nv_bfloat16*)pre_s, (const __nv_bfloat16*)post_s, (const __nv_bfloat16*)res_s,
                   (const __nv_bfloat16*)w_in, (__nv_bfloat16*)x_in, (__nv_bfloat16*)h, (uint8_t*)xrec_h, post, res, D, iters, eps};
    return (int)vk_launch(mhc_mix_norm_kernel, dim3(B), dim3(row_threads(D)), 0, stream, p);
}

// descriptor + call index -> kernel argument; a null descriptor (or world 1) means no exchange
static int ar_call(const vk_ar_desc* ar, int call, int B, int D, VkArCall* out) {
    *out = VkArCall{};
    if (ar == nullptr || ar->world <= 1) return VK_OK;
    if (ar->world > kArMaxWorld || ar->rank < 0 || ar->rank >= ar->world || B > ar->rows || ar->row_elems != D ||
        call < 0 || call >= ar->calls_per_step || ar->step == nullptr)
        return VK_EINVAL;
    out->d.world = ar->world; out->d.rank = ar->rank; out->d.rows = ar->rows; out->d.calls_per_step = ar->calls_per_step;
    out->d.spin_limit = ar->spin_limit;
    for (int p = 0; p < ar->world; p++) {
        if (ar->slots[p] == nullptr) return VK_EINVAL;
        out->d.slots[p] = (uint8_t*)ar->slots[p];
    }
    out->d.step = ar->step;
    out->call = call;
    return VK_OK;
}

int vk_add_rmsnorm_ar(const void* x, void* r, const void* w, void* h2, void* hn, void* xrec_hn, int B, int D, float eps,
                      int offset, const vk_ar_desc* ar, int call, cudaStream_t stream) {
    if (B <= 0 || D <= 0 || D % 8 != 0 || (xrec_hn != nullptr && (D % 64 != 0 || B > 16))) return VK_EINVAL;
    VkArCall a;
    if (ar_call(r != nullptr ? ar : nullptr, call, B, D, &a) != VK_OK) return VK_EINVAL;
    return (int)vk_launch(add_rmsnorm_kernel, dim3(B), dim3(row_threads(D)), 0, stream, (const __nv_bfloat16*)x,
                          (const __nv_bfloat16*)r, (const __nv_bfloat16*)w, (__nv_bfloat16*)h2, (__nv_bfloat16*)hn,
                          (uint8_t*)xrec_hn, D, eps, offset ? 1.f : 0.f, a);
}

int vk_add_rmsnorm(const void* x, const void* r, const void* w, void* h2, void* hn, void* xrec_hn, int B, int D, float eps,
                   int offset, cudaStream_t stream) {
    return vk_add_rmsnorm_ar(x, const_cast<void*>(r), w, h2, hn, xrec_hn, B, D, eps, offset, nullptr, 0, stream);
}

int vk_silu_mul(const void* gu, void* act, void* xrec_act, int B, int I, int ld_gu, cudaStream_t stream) {
    if (B <= 0 || I <= 0 || I % 64 != 0 || ld_gu % 8 != 0 || (xrec_act != nullptr && B > 16)) return VK_EINVAL;
    return (int)vk_launch(silu_mul_kernel, dim3((I / 8 + 255) / 256, B), dim3(256), 0, stream, (const __nv_bfloat16*)gu,
                          (__nv_bfloat16*)act, (uint8_t*)xrec_act, I, ld_gu);
}

int vk_engram_gather(const void* const* tables, const int* ld_table, const int* col0, const int* rows, const void* w,
                     void* e, int B, int n_orders, int dim, float eps, cudaStream_t stream) {
    if (B <= 0 || n_orders <= 0 || n_orders > 4) return VK_EINVAL;
    EngramGatherParams p = {};
    for (int i = 0; i < n_orders; i++) {
        p.tables[i] = (const __nv_bfloat16*)tables[i];
        p.ld_table[i] = ld_table[i];
        p.col0[i] = col0[i];
    }
    p.rows = rows; p.w = (const __nv_bfloat16*)w; p.e = (__nv_bfloat16*)e; p.n_orders = n_orders; p.dim = dim; p.eps = eps;
    return (int)vk_launch(engram_gather_kernel, dim3(B), dim3(kEwThreads), 0, stream, p);
}

int vk_mhc_combine_norm_ar(void* H, const void* h2, void* m, const void* x_in, const float* post, const float* res,
                           const void* w_next, void* hn, const void* eng_val, const void* eng_gate_w, const void* eng_gate_b,
                           void* y_out, int B, int D, int final_norm, float eps, const vk_ar_desc* ar, int call,
                           cudaStream_t stream) {
    if (B <= 0 || D <= 0 || D % 8 != 0) return VK_EINVAL;
    CombineParams p = {(__nv_bfloat16*)H, (const __nv_bfloat16*)h2, (const __nv_bfloat16*)m, (const __nv_bfloat16*)x_in,
                       post, res, (const __nv_bfloat16*)w_next, (__nv_bfloat16*)hn, (const __nv_bfloat16*)eng_val,
                       (const __nv_bfloat16*)eng_gate_w, (const __nv_bfloat16*)eng_gate_b, (__nv_bfloat16*)y_out, D,
                       final_norm, eps, VkArCall{}};
    if (ar_call(ar, call, B, D, &p.ar) != VK_OK) return VK_EINVAL;
    return (int)vk_launch(mhc_combine_norm_kernel, dim3(B), dim3(row_threads(D)), 0, stream, p);
}

int vk_mhc_combine_norm(void* H, const void* h2, const void* m, const void* x_in, const float* post, const float* res,
                        const void* w_next, void* hn, const void* eng_val, const void* eng_gate_w, const void* eng_gate_b,
                        void* y_out, int B, int D, int final_norm, float eps, cudaStream_t stream) {
    return vk_mhc_combine_norm_ar(H, h2, const_cast<void*>(m), x_in, post, res, w_next, hn, eng_val, eng_gate_w, eng_gate_b,
                                  y_out, B, D, final_norm, eps, nullptr, 0, stream);
}

// mhc_combine_norm of one layer + mhc_mix_norm of the next in one launch (see mhc_boundary_kernel). D / 8 <= 640.
int vk_mhc_boundary_ar(void* H, const void* h2, void* m, void* x_in, float* post, float* res, const void* w_next,
                       const void* eng_val, const void* eng_gate_w, const void* eng_gate_b, const void* w_dyn, const void* pre_s,
                       const void* post_s, const void* res_s, const void* w_in, void* h, void* xrec_h, int B, int D, int iters,
                       float eps, const vk_ar_desc* ar, int call, cudaStream_t stream) {
    if (B <= 0 || D <= 0 || D % 64 != 0 || D / 8 > kBoundaryThreads || (xrec_h != nullptr && B > 16)) return VK_EINVAL;
    BoundaryParams q = {};
    q.c = {(__nv_bfloat16*)H, (const __nv_bfloat16*)h2, (const __nv_bfloat16*)m, (const __nv_bfloat16*)x_in, post, res,
           (const __nv_bfloat16*)w_next, nullptr, (const __nv_bfloat16*)eng_val, (const __nv_bfloat16*)eng_gate_w,
           (const __nv_bfloat16*)eng_gate_b, nullptr, D, 0, eps, VkArCall{}};
    if (ar_call(ar, call, B, D, &q.c.ar) != VK_OK) return VK_EINVAL;
    q.w_dyn = (const __nv_bfloat16*)w_dyn; q.pre_s = (const __nv_bfloat16*)pre_s; q.post_s = (const __nv_bfloat16*)post_s;
    q.res_s = (const __nv_bfloat16*)res_s; q.w_in = (const __nv_bfloat16*)w_in; q.x_in_out = (__nv_bfloat16*)x_in;
    q.h = (__nv_bfloat16*)h; q.xrec_h = (uint8_t*)xrec_h; q.post_out = post; q.res_out = res; q.iters = iters;
    // a cluster of four CTAs per row when the row's pieces split into four whole x-record groups per CTA
    if (g_boundary_cluster && D % 256 == 0 && (D / 32) % 32 == 0)
        return (int)vk_launch_cluster(mhc_boundary_kernel<4>, dim3(B * 4), dim3(D / 32), 4, 0, stream, q);
    const int threads = ((D / 8 + 31) / 32) * 32;
    return (int)vk_launch(mhc_boundary_kernel<1>, dim3(B), dim3(threads), 0, stream, q);
}

int vk_mhc_boundary(void* H, const void* h2, const void* m, void* x_in, float* post, float* res, const void* w_next,
                    const void* eng_val, const void* eng_gate_w, const void* eng_gate_b, const void* w_dyn, const void* pre_s,
                    const void* post_s, const void* res_s, const void* w_in, void* h, void* xrec_h, int B, int D, int iters,
                    float eps, cudaStream_t stream) {
    return vk_mhc_boundary_ar(H, h2, const_cast<void*>(m), x_in, post, res, w_next, eng_val, eng_gate_w, eng_gate_b, w_dyn,
                              pre_s, post_s, res_s, w_in, h, xrec_h, B, D, iters, eps, nullptr, 0, stream);
}

int vk_bf16_gemm(const void* x, int ldx, const void* W, const void* bias, void* y, int ldy, int M, int N, int K,
                 cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0 || K % 8 != 0 || ldx % 8 != 0) return VK_EINVAL;
    for (int m0 = 0; m0 < M; m0 += 16) {
        const int m = M - m0 < 16 ? M - m0 : 16;
        const __nv_bfloat16* xp = (const __nv_bfloat16*)x + (size_t)m0 * ldx;
        __nv_bfloat16* yp = (__nv_bfloat16*)y + (size_t)m0 * ldy;
        cudaError_t e;
        if (m <= 4)
            e = vk_launch(bf16_gemm_rows_kernel<4>, dim3((N + 7) / 8), dim3(256), 0, stream, xp, ldx,
                          (const __nv_bfloat16*)W, (const __nv_bfloat16*)bias, yp, ldy, m, N, K);
        else
            e = vk_launch(bf16_gemm_rows_kernel<16>, dim3((N + 7) / 8), dim3(256), 0, stream, xp, ldx,
                          (const __nv_bfloat16*)W, (const __nv_bfloat16*)bias, yp, ldy, m, N, K);
        if (e != cudaSuccess) return (int)e;
    }
    return VK_OK;
}

int vk_argmax(const void* logits, int ld, int valid, int* out, int B, cudaStream_t stream) {
    if (B <= 0 || valid <= 0) return VK_EINVAL;
    return (int)vk_launch(argmax_kernel, dim3(B), dim3(1024), 0, stream, (const __nv_bfloat16*)logits, ld, valid, out);
}

}  // extern "C"
