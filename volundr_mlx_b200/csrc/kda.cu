// Kimi Delta Attention decode step, one CTA per (value head, row): depthwise causal conv (k = 4) + SiLU of this
// head's q / k / v channels, q/k l2 normalisation, the per-channel decay g and beta, the gated-delta-rule update of
// the fp32 state S[Dv, Dk] (read once, written once), y = S q, and the z-gated RMSNorm of y.
//
// Replaces, for L = 1, KDA.__call__ (volundr.py:388-439): DF.kda_conv_gates (decode_fused.py:362-493) ->
// kernels.gated_delta_vec (kernels.py:374-458) -> kernels.gated_norm (kernels.py:890-928), and the two small bf16
// linears in front of them (in_proj_b, f_up; volundr.py:392-393). Arithmetic per (b, hv), key head hk = hv / (HV/Hk):
//   c = sum_j x[t-3+j] * w[j] (fp32, products and sums rounded separately, j = 0..3); s = bf16(c * sigmoid(c))
//   q^ = s_q / sqrt(sum s_q^2 + 1e-6) * Dk^-1/2 ; k^ = s_k / sqrt(sum s_k^2 + 1e-6) ; v = s_v
//   g = exp(-exp(A_log) * softplus(a + dt_bias)), a = bf16(f_up . f_down(h)) ; beta = sigmoid(bf16(in_proj_b . h))
//   S <- S * g (per column) ; delta = (v - S k^) beta ; S <- S + delta (x) k^ ; y = S q^
//   out = bf16(w * (bf16(y) * rsqrt(mean bf16(y)^2 + eps)) * silu(z))
// State layout: fp32 [slot, HV, Dv, Dk], row = value dim, Dk contiguous (volundr.py:406). Dk = Dv = 128.
#include "common.cuh"
#include "xrec.cuh"

namespace {

struct KdaParams {
    const __nv_bfloat16* proj;     // [B, ldp]: q (Hk*128) | k (Hk*128) | v (HV*128) at 0, z at off_z, f_down at off_fd
    const __nv_bfloat16* h;        // [B, D] layer input (for in_proj_b)
    const __nv_bfloat16* w_b;      // [HV, D]
    const __nv_bfloat16* w_fup;    // packed by vk_kda_pack_fup: [HV][rank / 8][128][8]
    const float* conv_w;           // [C, 4]
    const float* A_log;            // [HV]
    const float* dt_bias;          // [HV*128]
    const __nv_bfloat16* norm_w;   // [128]
    __nv_bfloat16* conv;           // [2, slots, 3, C]: buffer *parity holds the state before the step, the other one
                                   // receives the state after it (two buffers: value heads that share a key head
                                   // read its q / k channels while one of them writes the new rows)
    const int* parity;             // device word, flipped at the end of every step
    size_t conv_stride;            // elements between the two buffers
    float* S;                      // [slots, HV, 128, 128]
    __nv_bfloat16* out;            // [B, HV*128]
    uint8_t* xrec_out;             // null, or HV * 2 x records receiving out
    int ldp, off_z, off_fd, D, Hk, HV, rank;
    float eps;
};

constexpr int kBdotPieces = 5;   // 16-byte pieces of the in_proj_b row a thread keeps in registers (hidden <= 5120)

__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// sum of three values over the 128-thread block in one pass: xor tree per warp, then warps 0..3 in order (the order
// of block_sum<4>)
__device__ __forceinline__ void block_sum3(float& a, float& b, float& c, float (*red3)[4]) {
    a = warp_sum(a); b = warp_sum(b); c = warp_sum(c);
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) { red3[0][warp] = a; red3[1][warp] = b; red3[2][warp] = c; }
    __syncthreads();
    a = ((red3[0][0] + red3[0][1]) + red3[0][2]) + red3[0][3];
    b = ((red3[1][0] + red3[1][1]) + red3[1][2]) + red3[1][3];
    c = ((red3[2][0] + red3[2][1]) + red3[2][2]) + red3[2][3];
}

__global__ void __launch_bounds__(128, 5) kda_step_kernel(const KdaParams p) {
    __shared__ float red[4];
    __shared__ float red3[3][4];
    __shared__ __align__(16) float qs[128], ks[128], gs[128], ys[128];
    __shared__ float vs[128];
    __shared__ float fd[256];
    // the state streams through a ring of two 8-row batches per warp: every lane copies (cp.async) and later reads
    // only its own 16 bytes of a row, so the ring needs no barrier
    __shared__ __align__(16) float ring[4][2][8][128];
    pdl_launch_dependents();   // (the dependent, a GEMM, reads only weights in front of its own wait)
    const int hv = blockIdx.x, b = blockIdx.y;
    VK_TS(1, 0);
    const int c = threadIdx.x, lane = c & 31, warp = c >> 5;
    const int rep = p.HV / p.Hk, hk = hv / rep;
    const int KD = p.Hk * 128, C = 2 * KD + p.HV * 128;
    const int ch[3] = {hk * 128 + c, KD + hk * 128 + c, 2 * KD + hv * 128 + c};
    // weights depend on no earlier kernel: fetch the small ones (conv taps, this thread's pieces of the in_proj_b
    // row), and start the head's f_up block towards L2, while the kernel before this one is still running
    const uint4* fup = reinterpret_cast<const uint4*>(p.w_fup) + (size_t)hv * (p.rank / 8) * 128 + c;
    if (c == 32) l2_prefetch_bulk(p.w_fup + (size_t)hv * 128 * p.rank, 128u * (uint32_t)p.rank * 2u);
    float4 cw[3];
#pragma unroll
    for (int i = 0; i < 3; i++) cw[i] = *reinterpret_cast<const float4*>(p.conv_w + (size_t)ch[i] * 4);
    const float a_log = p.A_log[hv], dtb = p.dt_bias[hv * 128 + c], nw = bf2f(p.norm_w[c]);
    const __nv_bfloat16* wb = p.w_b + (size_t)hv * p.D;
    uint4 wbv[kBdotPieces];
#pragma unroll
    for (int i = 0; i < kBdotPieces; i++) {
        const int k = c * 8 + i * 1024;
        wbv[i] = k < p.D ? *reinterpret_cast<const uint4*>(wb + k) : make_uint4(0u, 0u, 0u, 0u);
    }
    // Also in front of the wait: everything that kernels before the one in front of this launch wrote (the in_proj
    // GEMM, whose output alone this step waits for): the state, both conv buffers, the parity word, the layer input h.
    float* Sb = p.S + (((size_t)b * p.HV + hv) * 128) * 128;
    const int par_word = *p.parity;
    const __nv_bfloat16* hb = p.h + (size_t)b * p.D;
    uint4 hx[kBdotPieces];
#pragma unroll
    for (int i = 0; i < kBdotPieces; i++) {
        const int k = c * 8 + i * 1024;
        hx[i] = k < p.D ? *reinterpret_cast<const uint4*>(hb + k) : make_uint4(0u, 0u, 0u, 0u);
    }
    __nv_bfloat16 cx[3][4], cy[3][3];
#pragma unroll
    for (int i = 0; i < 3; i++) {
        const size_t cb = (size_t)b * 3 * C + ch[i];
        const __nv_bfloat16* c0 = p.conv + cb;
        const __nv_bfloat16* c1 = p.conv + p.conv_stride + cb;
        cx[i][0] = c0[0]; cx[i][1] = c0[C]; cx[i][2] = c0[2 * (size_t)C];
        cy[i][0] = c1[0]; cy[i][1] = c1[C]; cy[i][2] = c1[2 * (size_t)C];
    }
#pragma unroll
    for (int bt = 0; bt < 2; bt++) {
#pragma unroll
        for (int i = 0; i < 8; i++)
            cp_async16(&ring[warp][bt][i][4 * lane], Sb + (size_t)(warp * 32 + bt * 8 + i) * 128 + 4 * lane);
        cp_async_commit();
    }
    pdl_wait();
    VK_TS(1, 1);
    const __nv_bfloat16* pr = p.proj + (size_t)b * p.ldp;
#pragma unroll
    for (int i = 0; i < 3; i++) cx[i][3] = pr[ch[i]];
    const float z = bf2f(pr[p.off_z + hv * 128 + c]);
    for (int i = c; i < p.rank; i += 128) fd[i] = bf2f(pr[p.off_fd + i]);

    // ---- beta's dot product
    float bdot = 0.f;
#pragma unroll
    for (int i = 0; i < kBdotPieces; i++) {
        const uint4 wv = wbv[i], xv = hx[i];
        bdot = fmaf(bf_lo(wv.x), bf_lo(xv.x), bdot); bdot = fmaf(bf_hi(wv.x), bf_hi(xv.x), bdot);
        bdot = fmaf(bf_lo(wv.y), bf_lo(xv.y), bdot); bdot = fmaf(bf_hi(wv.y), bf_hi(xv.y), bdot);
        bdot = fmaf(bf_lo(wv.z), bf_lo(xv.z), bdot); bdot = fmaf(bf_hi(wv.z), bf_hi(xv.z), bdot);
        bdot = fmaf(bf_lo(wv.w), bf_lo(xv.w), bdot); bdot = fmaf(bf_hi(wv.w), bf_hi(xv.w), bdot);
    }
    for (int k = c * 8 + kBdotPieces * 1024; k < p.D; k += 1024) {   // (hidden sizes beyond 8192)
        const uint4 wv = *reinterpret_cast<const uint4*>(wb + k);
        const uint4 xv = *reinterpret_cast<const uint4*>(hb + k);
        bdot = fmaf(bf_lo(wv.x), bf_lo(xv.x), bdot); bdot = fmaf(bf_hi(wv.x), bf_hi(xv.x), bdot);
        bdot = fmaf(bf_lo(wv.y), bf_lo(xv.y), bdot); bdot = fmaf(bf_hi(wv.y), bf_hi(xv.y), bdot);
        bdot = fmaf(bf_lo(wv.z), bf_lo(xv.z), bdot); bdot = fmaf(bf_hi(wv.z), bf_hi(xv.z), bdot);
        bdot = fmaf(bf_lo(wv.w), bf_lo(xv.w), bdot); bdot = fmaf(bf_hi(wv.w), bf_hi(xv.w), bdot);
    }
    VK_TS(1, 2);
    // f_up arrives packed (vk_kda_pack_fup): [head][rank / 8][channel][8], so that the 128 channels of a head read
    // consecutive 16-byte pieces. The first 64 ranks are requested here, to arrive during the conv and its reduction.
    uint4 fw[8];
#pragma unroll
    for (int u = 0; u < 8; u++) fw[u] = 8 * u < p.rank ? fup[(size_t)u * 128] : make_uint4(0u, 0u, 0u, 0u);

    // ---- conv + SiLU of this head's q, k, v channel c; new conv state
    const int par = par_word & 1;
    __nv_bfloat16* conv_out = p.conv + (size_t)(1 - par) * p.conv_stride;
    if (par) {
#pragma unroll
        for (int i = 0; i < 3; i++) { cx[i][0] = cy[i][0]; cx[i][1] = cy[i][1]; cx[i][2] = cy[i][2]; }
    }
    float s3[3];
#pragma unroll
    for (int i = 0; i < 3; i++) {
        const size_t cb = (size_t)b * 3 * C + ch[i];
        float acc = __fmul_rn(bf2f(cx[i][0]), cw[i].x);
        acc = __fadd_rn(acc, __fmul_rn(bf2f(cx[i][1]), cw[i].y));
        acc = __fadd_rn(acc, __fmul_rn(bf2f(cx[i][2]), cw[i].z));
        acc = __fadd_rn(acc, __fmul_rn(bf2f(cx[i][3]), cw[i].w));
        s3[i] = bfr(acc / (1.f + expf(-acc)));
        if (i == 2 || hv % rep == 0) {
            conv_out[cb] = cx[i][1];
            conv_out[cb + C] = cx[i][2];
            conv_out[cb + 2 * (size_t)C] = cx[i][3];
        }
    }
    float ssq = s3[0] * s3[0], ssk = s3[1] * s3[1];
    VK_TS(1, 3);
    block_sum3(ssq, ssk, bdot, red3);   // (its barrier also publishes fd)
    qs[c] = (s3[0] / sqrtf(ssq + 1e-6f)) * 0.08838834764831845f;  // 128^-1/2
    ks[c] = s3[1] / sqrtf(ssk + 1e-6f);
    vs[c] = s3[2];
    VK_TS(1, 4);

    // ---- decay g[c] and beta
    {
        float a = 0.f;
        for (int r0 = 0; r0 < p.rank; r0 += 64) {
            uint4 nx[8];   // the next 64 ranks, requested before this batch is used
#pragma unroll
            for (int u = 0; u < 8; u++)
                nx[u] = r0 + 64 + 8 * u < p.rank ? fup[(size_t)((r0 + 64) / 8 + u) * 128] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int u = 0; u < 8; u++) {
                if (r0 + 8 * u < p.rank) {
                    const int r = r0 + 8 * u;
                    a = fmaf(bf_lo(fw[u].x), fd[r], a); a = fmaf(bf_hi(fw[u].x), fd[r + 1], a);
                    a = fmaf(bf_lo(fw[u].y), fd[r + 2], a); a = fmaf(bf_hi(fw[u].y), fd[r + 3], a);
                    a = fmaf(bf_lo(fw[u].z), fd[r + 4], a); a = fmaf(bf_hi(fw[u].z), fd[r + 5], a);
                    a = fmaf(bf_lo(fw[u].w), fd[r + 6], a); a = fmaf(bf_hi(fw[u].w), fd[r + 7], a);
                }
            }
#pragma unroll
            for (int u = 0; u < 8; u++) fw[u] = nx[u];
        }
        a = bfr(a);
        gs[c] = expf(-expf(a_log) * softplus_f(a + dtb));
    }
    bdot = bfr(bdot);
    const float beta = 1.f / (1.f + expf(-bdot));
    __syncthreads();   // qs / ks / gs / vs
    VK_TS(1, 5);
    const float4 g4 = *reinterpret_cast<const float4*>(gs + 4 * lane);

    // ---- recurrence: warp w owns rows 32 w .. 32 w + 31 of S; lane l columns 4 l .. 4 l + 3
    const float4 k4 = *reinterpret_cast<const float4*>(ks + 4 * lane);
    const float4 q4 = *reinterpret_cast<const float4*>(qs + 4 * lane);
#pragma unroll 1
    for (int bt = 0; bt < 4; bt++) {
        const int r0 = warp * 32 + bt * 8;
        cp_async_wait1();   // every group but the newest has landed: batch bt is in the ring
        float4 s[8];
#pragma unroll
        for (int i = 0; i < 8; i++) s[i] = *reinterpret_cast<const float4*>(&ring[warp][bt & 1][i][4 * lane]);
        if (bt + 2 < 4) {
#pragma unroll
            for (int i = 0; i < 8; i++)
                cp_async16(&ring[warp][bt & 1][i][4 * lane], Sb + (size_t)(r0 + 16 + i) * 128 + 4 * lane);
        }
        cp_async_commit();   // (an empty group in the last two rounds keeps the count uniform)
        VK_TS(1, 6 + bt);
        float kv[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            s[i].x *= g4.x; s[i].y *= g4.y; s[i].z *= g4.z; s[i].w *= g4.w;
            kv[i] = fmaf(s[i].w, k4.w, fmaf(s[i].z, k4.z, fmaf(s[i].y, k4.y, s[i].x * k4.x)));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int i = 0; i < 8; i++) kv[i] += __shfl_xor_sync(0xffffffffu, kv[i], o);
        float y[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float d = (vs[r0 + i] - kv[i]) * beta;
            s[i].x = fmaf(d, k4.x, s[i].x); s[i].y = fmaf(d, k4.y, s[i].y);
            s[i].z = fmaf(d, k4.z, s[i].z); s[i].w = fmaf(d, k4.w, s[i].w);
            y[i] = fmaf(s[i].w, q4.w, fmaf(s[i].z, q4.z, fmaf(s[i].y, q4.y, s[i].x * q4.x)));
            *reinterpret_cast<float4*>(Sb + (size_t)(r0 + i) * 128 + 4 * lane) = s[i];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int i = 0; i < 8; i++) y[i] += __shfl_xor_sync(0xffffffffu, y[i], o);
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < 8; i++) ys[r0 + i] = y[i];
        }
    }
    __syncthreads();

    // ---- gated norm over the value head
    VK_TS(1, 10);
    const float yb = bfr(ys[c]);
    const float ss = block_sum<4>(yb * yb, red);
    const float inv = rsqrtf(ss * (1.f / 128.f) + p.eps);
    const float ov = bfr(((yb * inv) * nw) * (z / (1.f + expf(-z))));
    p.out[(size_t)b * p.HV * 128 + hv * 128 + c] = f2bf(ov);
    if (p.xrec_out != nullptr) {
        // this head fills two 64-column groups: element stores, group sums = warp xor tree, then warp 2g + warp 2g+1
        const int kg = hv * 2 + (c >> 6);
        *xrec_elem(p.xrec_out, kg, b, c & 63) = f2bf(ov);
        const float ws = warp_sum(ov);
        __syncthreads();
        if (lane == 0) red[warp] = ws;
        __syncthreads();
        if ((c & 63) == 0) xrec_store_sum(p.xrec_out, kg, b, red[warp] + red[warp + 1]);
    }
    VK_TS(1, 11);
}

}  // namespace

// ------------------------------------------------------------------------------------------------ T tokens per row
// The same recurrence over a chunk of T tokens per row in one launch: the prefill form (kernels.gated_delta_tg,
// kernels.py:544-555) and the verify / commit-replay form (verify._kda, spec/verify.py:33-53; batch_spec.py:186-195).
// One CTA per (value head, row): half of its threads keep the state S[Dv, Dk] in registers for the whole chunk (the
// state is read once and written once per launch, however many tokens there are) and run the recurrence, the other half
// does the per-token work around it, one token group ahead and one behind. Tokens go through in groups of kChunkTok:
// (A) conv + SiLU, norms, decay and beta of the group's tokens, (B) the recurrence, token after token (every row dot is
// formed as 32 four-element fma chains combined in the order of a warp's xor tree: the sums, and so every bit of the
// result, are those of kda_step_kernel), (C) the gated norm of the group's outputs. `accept[b]` (optional) ends row b's
// chunk early: later tokens leave state, conv window and output alone (the commit of a verify step: only the accepted
// prefix is replayed).
constexpr int kChunkTok = 8;

struct KdaChunkParams {
    KdaParams k;          // proj / h / out rows are (b * T + t); xrec_out unused
    const int* accept;    // [B] or null
    const int* row_off;   // [B] or null: first row of request b in proj / h / out (null: b * T)
    int T;
    int write_state;      // 0: outputs only, the state and the conv window stay as they were (a verify pass)
};

// xor-tree sum of p[0..31] as the 32 lanes of a warp would form it
__device__ __forceinline__ float tree32(float (&p)[32]) {
#pragma unroll
    for (int l = 0; l < 16; l++) p[l] += p[l + 16];
#pragma unroll
    for (int l = 0; l < 8; l++) p[l] += p[l + 8];
#pragma unroll
    for (int l = 0; l < 4; l++) p[l] += p[l + 4];
    p[0] += p[2]; p[1] += p[3];
    return p[0] + p[1];
}

// Shared memory of kda_chunk_kernel (dynamic: more than the 48 KB a kernel gets without asking).
struct KdaChunkSmem {
    float qs[2][kChunkTok][128], ks[2][kChunkTok][128], gs[2][kChunkTok][128], vs[2][kChunkTok][128];   // per group, two buffers
    float ys[2][kChunkTok][128];        // the recurrence's outputs, for the gated norm one group later
    float betas[2][kChunkTok];
    float fd[kChunkTok][256];
    float red[4 * kChunkTok][4];
};

// One named barrier per front group (128 threads each): ids 1 and 2 (0 is __syncthreads).
__device__ __forceinline__ void front_barrier(int group) {
    if (group == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
    else asm volatile("bar.sync 2, 128;" ::: "memory");
}

// 512 threads. The "back" half (threads 0..255) owns the state and runs the recurrence of token group g while the two
// "front" groups (threads 256..383 and 384..511) prepare group g + 1 (conv + SiLU, norms, decay, beta) and finish
// group g - 1 (gated norm, output), each for its own four of the group's eight tokens, so only the recurrence itself
// lies on the critical path of a row's tokens. Every sum is formed in the order of kda_step_kernel: per-channel work by
// channel c = thread index within its front group (warp sums over 32 channels, the four warps' sums added in order),
// the recurrence's row dots as 32 four-column chains combined in the order of a warp's xor tree.
__global__ void __launch_bounds__(512, 1) kda_chunk_kernel(const KdaChunkParams cp) {
    const KdaParams& p = cp.k;
    extern __shared__ __align__(16) uint8_t kda_chunk_smem[];
    KdaChunkSmem& sm = *reinterpret_cast<KdaChunkSmem*>(kda_chunk_smem);
    pdl_launch_dependents();
    const int hv = blockIdx.x, b = blockIdx.y;
    const int T = cp.T;

    if (threadIdx.x < 256) {
        // ------------------------------------------------------------------------------------------ the recurrence
        // Thread (vg, j) = (c >> 3, c & 7) keeps, of the four state rows 4 vg .. 4 vg + 3, the columns of the four
        // four-column chains l = j + 8 i. The xor tree's first two levels (l +- 16, 8) stay inside the thread, the last
        // three (l +- 4, 2, 1) are three shuffles between the eight threads of the rows. A thread so reads an eighth
        // of q / k / g per token: shared-memory traffic, not arithmetic, bounds a one-thread-per-row form.
        const int c = threadIdx.x, j8 = c & 7, vg = c >> 3;
        pdl_wait();
        const int n_tok = cp.accept != nullptr ? min(max(cp.accept[b], 0), T) : T;
        const int n_grp = (n_tok + kChunkTok - 1) / kChunkTok;
        float* Sbase = p.S + (((size_t)b * p.HV + hv) * 128 + 4 * vg) * 128;
        float st[4][4][4];
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float4 v4 = *reinterpret_cast<const float4*>(Sbase + r * 128 + 4 * (j8 + 8 * i));
                st[r][i][0] = v4.x; st[r][i][1] = v4.y; st[r][i][2] = v4.z; st[r][i][3] = v4.w;
            }
        VK_TS(4, 0);
        __syncthreads();                                   // group 0 is prepared
        VK_TS(4, 1);
        for (int g = 0; g < n_grp; g++) {
            const int buf = g & 1;
            const int nt = min(kChunkTok, n_tok - g * kChunkTok);
            for (int tt = 0; tt < nt; tt++) {
                const float beta = sm.betas[buf][tt];
                const float4 v4 = *reinterpret_cast<const float4*>(&sm.vs[buf][tt][4 * vg]);
                const float vv[4] = {v4.x, v4.y, v4.z, v4.w};
                float pp[4][4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int l = j8 + 8 * i;
                    const float4 g4 = *reinterpret_cast<const float4*>(&sm.gs[buf][tt][4 * l]);
                    const float4 k4 = *reinterpret_cast<const float4*>(&sm.ks[buf][tt][4 * l]);
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        st[r][i][0] *= g4.x; st[r][i][1] *= g4.y; st[r][i][2] *= g4.z; st[r][i][3] *= g4.w;
                        pp[r][i] = fmaf(st[r][i][3], k4.w, fmaf(st[r][i][2], k4.z, fmaf(st[r][i][1], k4.y, st[r][i][0] * k4.x)));
                    }
                }
                float d[4];
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    pp[r][0] += pp[r][2]; pp[r][1] += pp[r][3];                  // l + 16
                    float x = pp[r][0] + pp[r][1];                               // l + 8
                    x += __shfl_xor_sync(0xffffffffu, x, 4);                     // l + 4
                    x += __shfl_xor_sync(0xffffffffu, x, 2);                     // l + 2
                    x += __shfl_xor_sync(0xffffffffu, x, 1);                     // l + 1
                    d[r] = (vv[r] - x) * beta;
                }
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int l = j8 + 8 * i;
                    const float4 k4 = *reinterpret_cast<const float4*>(&sm.ks[buf][tt][4 * l]);
                    const float4 q4 = *reinterpret_cast<const float4*>(&sm.qs[buf][tt][4 * l]);
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        st[r][i][0] = fmaf(d[r], k4.x, st[r][i][0]); st[r][i][1] = fmaf(d[r], k4.y, st[r][i][1]);
                        st[r][i][2] = fmaf(d[r], k4.z, st[r][i][2]); st[r][i][3] = fmaf(d[r], k4.w, st[r][i][3]);
                        pp[r][i] = fmaf(st[r][i][3], q4.w, fmaf(st[r][i][2], q4.z, fmaf(st[r][i][1], q4.y, st[r][i][0] * q4.x)));
                    }
                }
                float o[4];
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    pp[r][0] += pp[r][2]; pp[r][1] += pp[r][3];
                    float x = pp[r][0] + pp[r][1];
                    x += __shfl_xor_sync(0xffffffffu, x, 4);
                    x += __shfl_xor_sync(0xffffffffu, x, 2);
                    x += __shfl_xor_sync(0xffffffffu, x, 1);
                    o[r] = x;
                }
                if (j8 == 0) *reinterpret_cast<float4*>(&sm.ys[buf][tt][4 * vg]) = make_float4(o[0], o[1], o[2], o[3]);
            }
            __syncthreads();                               // group g + 1 is prepared, ys of group g are in place
        }
        VK_TS(4, 2);
        if (cp.write_state) {
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int i = 0; i < 4; i++)
                    *reinterpret_cast<float4*>(Sbase + r * 128 + 4 * (j8 + 8 * i)) =
                        make_float4(st[r][i][0], st[r][i][1], st[r][i][2], st[r][i][3]);
        }
        return;
    }

    // ---------------------------------------------------------------------------------------------- the front groups
    const int fg = (threadIdx.x - 256) >> 7;             // this group's tokens of every token group: 4 fg .. 4 fg + 3
    const int c = threadIdx.x & 127, lane = c & 31, warp = c >> 5;
    const int rep = p.HV / p.Hk, hk = hv / rep;
    const int KD = p.Hk * 128, C = 2 * KD + p.HV * 128;
    const int ch[3] = {hk * 128 + c, KD + hk * 128 + c, 2 * KD + hv * 128 + c};
    const uint4* fup = reinterpret_cast<const uint4*>(p.w_fup) + (size_t)hv * (p.rank / 8) * 128 + c;
    float4 cw[3];
#pragma unroll
    for (int i = 0; i < 3; i++) cw[i] = *reinterpret_cast<const float4*>(p.conv_w + (size_t)ch[i] * 4);
    const float a_log = p.A_log[hv], dtb = p.dt_bias[hv * 128 + c], nw = bf2f(p.norm_w[c]);
    const __nv_bfloat16* wb = p.w_b + (size_t)hv * p.D;
    pdl_wait();
    const int n_tok = cp.accept != nullptr ? min(max(cp.accept[b], 0), T) : T;
    const int n_grp = (n_tok + kChunkTok - 1) / kChunkTok;
    const size_t row0 = cp.row_off != nullptr ? (size_t)cp.row_off[b] : (size_t)b * T;
    const int par = *p.parity & 1;
    const __nv_bfloat16* conv_in = p.conv + (size_t)par * p.conv_stride;
    __nv_bfloat16* conv_out = p.conv + (size_t)(1 - par) * p.conv_stride;
    // input of channel kind i at chunk position tau: a row of proj, or (tau < 0) the conv window in front of the chunk
    auto xin = [&](int i, int tau) -> __nv_bfloat16 {
        return tau >= 0 ? p.proj[(row0 + tau) * p.ldp + ch[i]] : conv_in[(size_t)b * 3 * C + ch[i] + (size_t)(3 + tau) * C];
    };
    constexpr int kFront = kChunkTok / 2;                  // tokens of a token group per front group

    // (A) of this front group's tokens of token group g, into buffer `buf`: conv + SiLU, the two norms, decay, beta
    auto prepare = [&](int g, int buf) {
        const int t0 = g * kChunkTok + kFront * fg;        // chunk position of the first of them
        const int nt = min(kFront, n_tok - t0);            // (<= 0: nothing to do but the barriers)
        if (nt > 0) {
            __nv_bfloat16 xs[3][kFront + 3];               // the inputs t0 - 3 .. t0 + 3 of the thread's three channels
#pragma unroll
            for (int i = 0; i < 3; i++)
#pragma unroll
                for (int m = 0; m < kFront + 3; m++)
                    if (m < nt + 3) xs[i][m] = xin(i, t0 - 3 + m);
            float s3[kFront][3], bdot[kFront];
#pragma unroll
            for (int u = 0; u < kFront; u++) {
                bdot[u] = 0.f;
#pragma unroll
                for (int i = 0; i < 3; i++) {
                    s3[u][i] = 0.f;
                    if (u < nt) {
                        float acc = __fmul_rn(bf2f(xs[i][u]), cw[i].x);
                        acc = __fadd_rn(acc, __fmul_rn(bf2f(xs[i][u + 1]), cw[i].y));
                        acc = __fadd_rn(acc, __fmul_rn(bf2f(xs[i][u + 2]), cw[i].z));
                        acc = __fadd_rn(acc, __fmul_rn(bf2f(xs[i][u + 3]), cw[i].w));
                        s3[u][i] = bfr(acc / (1.f + expf(-acc)));
                    }
                }
            }
#pragma unroll
            for (int sb = 0; sb < kFront; sb += 2) {       // beta's dot and f_down, two tokens at a time
                uint4 hx[2][kBdotPieces];
                __nv_bfloat16 fdv[2][2];                   // rank <= 256: at most two f_down values per thread
#pragma unroll
                for (int v = 0; v < 2; v++) {
                    if (sb + v < nt) {
                        const size_t rowi = row0 + t0 + sb + v;
                        const __nv_bfloat16* hb = p.h + rowi * p.D;
#pragma unroll
                        for (int i = 0; i < kBdotPieces; i++) {
                            const int k = c * 8 + i * 1024;
                            hx[v][i] = k < p.D ? *reinterpret_cast<const uint4*>(hb + k) : make_uint4(0u, 0u, 0u, 0u);
                        }
#pragma unroll
                        for (int i = 0; i < 2; i++)
                            if (c + 128 * i < p.rank) fdv[v][i] = p.proj[rowi * p.ldp + p.off_fd + c + 128 * i];
                    }
                }
#pragma unroll
                for (int v = 0; v < 2; v++) {
                    const int u = sb + v, tt = kFront * fg + u;
                    if (u < nt) {
#pragma unroll
                        for (int i = 0; i < 2; i++)
                            if (c + 128 * i < p.rank) sm.fd[tt][c + 128 * i] = bf2f(fdv[v][i]);
                        float bd = 0.f;
#pragma unroll
                        for (int i = 0; i < kBdotPieces; i++) {
                            const int k = c * 8 + i * 1024;    // (the weight row's pieces stay in L1 from token to token)
                            const uint4 wv = k < p.D ? *reinterpret_cast<const uint4*>(wb + k) : make_uint4(0u, 0u, 0u, 0u);
                            const uint4 xv = hx[v][i];
                            bd = fmaf(bf_lo(wv.x), bf_lo(xv.x), bd); bd = fmaf(bf_hi(wv.x), bf_hi(xv.x), bd);
                            bd = fmaf(bf_lo(wv.y), bf_lo(xv.y), bd); bd = fmaf(bf_hi(wv.y), bf_hi(xv.y), bd);
                            bd = fmaf(bf_lo(wv.z), bf_lo(xv.z), bd); bd = fmaf(bf_hi(wv.z), bf_hi(xv.z), bd);
                            bd = fmaf(bf_lo(wv.w), bf_lo(xv.w), bd); bd = fmaf(bf_hi(wv.w), bf_hi(xv.w), bd);
                        }
                        const __nv_bfloat16* hb = p.h + (row0 + t0 + u) * p.D;
                        for (int k = c * 8 + kBdotPieces * 1024; k < p.D; k += 1024) {   // (hidden sizes beyond 5120)
                            const uint4 wv = *reinterpret_cast<const uint4*>(wb + k);
                            const uint4 xv = *reinterpret_cast<const uint4*>(hb + k);
                            bd = fmaf(bf_lo(wv.x), bf_lo(xv.x), bd); bd = fmaf(bf_hi(wv.x), bf_hi(xv.x), bd);
                            bd = fmaf(bf_lo(wv.y), bf_lo(xv.y), bd); bd = fmaf(bf_hi(wv.y), bf_hi(xv.y), bd);
                            bd = fmaf(bf_lo(wv.z), bf_lo(xv.z), bd); bd = fmaf(bf_hi(wv.z), bf_hi(xv.z), bd);
                            bd = fmaf(bf_lo(wv.w), bf_lo(xv.w), bd); bd = fmaf(bf_hi(wv.w), bf_hi(xv.w), bd);
                        }
                        bdot[u] = bd;
                        sm.qs[buf][tt][c] = s3[u][0]; sm.ks[buf][tt][c] = s3[u][1]; sm.vs[buf][tt][c] = s3[u][2];
                    }
                }
            }
            // the twelve warp sums of the four tokens, level by level (each sum is the xor tree of warp_sum)
            float ws[kFront][3];
#pragma unroll
            for (int u = 0; u < kFront; u++) { ws[u][0] = s3[u][0] * s3[u][0]; ws[u][1] = s3[u][1] * s3[u][1]; ws[u][2] = bdot[u]; }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int u = 0; u < kFront; u++)
#pragma unroll
                    for (int i = 0; i < 3; i++) ws[u][i] += __shfl_xor_sync(0xffffffffu, ws[u][i], o);
#pragma unroll
            for (int u = 0; u < kFront; u++) {
                const int tt = kFront * fg + u;
                if (u < nt && lane == 0) {
                    sm.red[3 * tt][warp] = ws[u][0]; sm.red[3 * tt + 1][warp] = ws[u][1]; sm.red[3 * tt + 2][warp] = ws[u][2];
                }
            }
        }
        front_barrier(fg);
        if (nt > 0) {
            // the decay's low-rank product for the four tokens at once: f_up is read once, and the tokens' fma chains
            // (each in the order of kda_step_kernel) run side by side
            float av[kFront];
#pragma unroll
            for (int u = 0; u < kFront; u++) av[u] = 0.f;
            uint4 wnext = fup[0];
            for (int r = 0; r < p.rank; r += 8) {
                const uint4 wv = wnext;
                if (r + 8 < p.rank) wnext = fup[(size_t)(r / 8 + 1) * 128];      // in flight while this piece is used
                const float w8[8] = {bf_lo(wv.x), bf_hi(wv.x), bf_lo(wv.y), bf_hi(wv.y), bf_lo(wv.z), bf_hi(wv.z), bf_lo(wv.w), bf_hi(wv.w)};
#pragma unroll
                for (int u = 0; u < kFront; u++) {
                    const int tt = kFront * fg + u;
                    const float4 f0 = *reinterpret_cast<const float4*>(&sm.fd[tt][r]);
                    const float4 f1 = *reinterpret_cast<const float4*>(&sm.fd[tt][r + 4]);
                    float a = av[u];
                    a = fmaf(w8[0], f0.x, a); a = fmaf(w8[1], f0.y, a); a = fmaf(w8[2], f0.z, a); a = fmaf(w8[3], f0.w, a);
                    a = fmaf(w8[4], f1.x, a); a = fmaf(w8[5], f1.y, a); a = fmaf(w8[6], f1.z, a); a = fmaf(w8[7], f1.w, a);
                    av[u] = a;
                }
            }
#pragma unroll
            for (int u = 0; u < kFront; u++) {
                const int tt = kFront * fg + u;
                if (u < nt) {
                    const float ssq = ((sm.red[3 * tt][0] + sm.red[3 * tt][1]) + sm.red[3 * tt][2]) + sm.red[3 * tt][3];
                    const float ssk = ((sm.red[3 * tt + 1][0] + sm.red[3 * tt + 1][1]) + sm.red[3 * tt + 1][2]) + sm.red[3 * tt + 1][3];
                    const float bd = ((sm.red[3 * tt + 2][0] + sm.red[3 * tt + 2][1]) + sm.red[3 * tt + 2][2]) + sm.red[3 * tt + 2][3];
                    sm.qs[buf][tt][c] = (sm.qs[buf][tt][c] / sqrtf(ssq + 1e-6f)) * 0.08838834764831845f;  // 128^-1/2
                    sm.ks[buf][tt][c] = sm.ks[buf][tt][c] / sqrtf(ssk + 1e-6f);
                    const float a = bfr(av[u]);
                    sm.gs[buf][tt][c] = expf(-expf(a_log) * softplus_f(a + dtb));
                    if (c == 0) sm.betas[buf][tt] = 1.f / (1.f + expf(-bfr(bd)));
                }
            }
        }
        front_barrier(fg);      // (fd and red of these tokens are free for the next token group)
    };

    // (C) of this front group's tokens of token group g: gated norm of the outputs the recurrence left in ys[buf]
    auto finish = [&](int g, int buf) {
        const int t0 = g * kChunkTok + kFront * fg;
        const int nt = min(kFront, n_tok - t0);
        float zv[kFront], yv[kFront], wy[kFront];
#pragma unroll
        for (int u = 0; u < kFront; u++) {                 // the gate inputs are fetched together
            zv[u] = 0.f;
            if (u < nt) zv[u] = bf2f(p.proj[(row0 + t0 + u) * p.ldp + p.off_z + hv * 128 + c]);
        }
#pragma unroll
        for (int u = 0; u < kFront; u++) {
            yv[u] = u < nt ? bfr(sm.ys[buf][kFront * fg + u][c]) : 0.f;
            wy[u] = yv[u] * yv[u];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < kFront; u++) wy[u] += __shfl_xor_sync(0xffffffffu, wy[u], o);
#pragma unroll
        for (int u = 0; u < kFront; u++)
            if (u < nt && lane == 0) sm.red[3 * kChunkTok + kFront * fg + u][warp] = wy[u];
        front_barrier(fg);
#pragma unroll
        for (int u = 0; u < kFront; u++) {
            if (u < nt) {
                const float* rr = sm.red[3 * kChunkTok + kFront * fg + u];
                float ss = 0.f;
                ss += rr[0]; ss += rr[1]; ss += rr[2]; ss += rr[3];
                const float inv = rsqrtf(ss * (1.f / 128.f) + p.eps);
                const float z = zv[u];
                const float ov = bfr(((yv[u] * inv) * nw) * (z / (1.f + expf(-z))));
                p.out[(row0 + t0 + u) * p.HV * 128 + hv * 128 + c] = f2bf(ov);
            }
        }
        front_barrier(fg);
    };

    if (n_grp > 0) prepare(0, 0);
    __syncthreads();                                       // group 0 is prepared
    for (int g = 0; g < n_grp; g++) {
        const int buf = g & 1;
        if (g + 1 < n_grp) prepare(g + 1, buf ^ 1);        // while the back half runs group g
        if (g > 0) finish(g - 1, buf ^ 1);
        __syncthreads();                                   // group g's outputs are in ys[buf]
    }
    if (n_grp > 0) finish(n_grp - 1, (n_grp - 1) & 1);
    if (!cp.write_state || fg != 0) return;
    // the conv window behind the chunk: the last three inputs of the thread's channels
#pragma unroll
    for (int i = 0; i < 3; i++) {
        if (i == 2 || hv % rep == 0) {
            const size_t cb = (size_t)b * 3 * C + ch[i];
#pragma unroll
            for (int m = 0; m < 3; m++) conv_out[cb + (size_t)m * C] = xin(i, n_tok - 3 + m);
        }
    }
}

// f_up [HV*128, rank] row-major (the checkpoint's layout) -> [HV][rank / 8][128][8]
__global__ void kda_pack_fup_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst, int HV, int rank) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)HV * 128 * rank;
    if (idx >= total) return;
    const int e = (int)(idx & 7);
    const int ch = (int)((idx >> 3) & 127);
    const size_t rest = idx >> 10;
    const int r8 = (int)(rest % (rank / 8)), hv = (int)(rest / (rank / 8));
    dst[idx] = src[((size_t)hv * 128 + ch) * rank + r8 * 8 + e];
}

extern "C" {

// The layout vk_kda_step reads f_up in (coalesced 16-byte pieces per channel). Once at load time.
int vk_kda_pack_fup(const void* src, void* dst, int HV, int rank, cudaStream_t stream) {
    if (HV <= 0 || rank <= 0 || rank % 8 != 0 || src == dst) return VK_EINVAL;
    const size_t total = (size_t)HV * 128 * rank;
    kda_pack_fup_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, HV, rank);
    return (int)cudaGetLastError();
}

// Five CTAs of 36 KB share an SM only with the largest shared-memory carve-out: ask for it once per device, outside
// any stream capture (a hint: the kernel is correct without it, only slower).
int vk_kda_configure(void) {
    VK_CUDA(cudaFuncSetAttribute(kda_step_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    return VK_OK;
}

// T tokens per row in one launch (prefill chunks; verify and its commit replay). Rows of proj / h / out are b * T + t,
// or row_offset[b] + t when row_offset is given (ragged chunks: request b has accept[b] <= T tokens of its own, the
// requests' rows lie one after another). accept (optional, [B]): row b stops after accept[b] tokens. The conv window
// after the chunk lands in the other buffer, as after one vk_kda_step: flip the parity word once per launch.
int vk_kda_chunk_ragged(const void* proj, int ldp, int off_z, int off_fd, const void* h, const void* w_b, const void* w_fup,
                        const float* conv_w, const float* A_log, const float* dt_bias, const void* norm_w, void* conv,
                        const int* parity, size_t conv_stride, float* S, void* out, const int* accept,
                        const int* row_offset, int write_state, int B, int T, int D, int Hk, int HV, int Dk, int Dv,
                        int rank, float eps, cudaStream_t stream) {
    if (B <= 0 || T <= 0 || Dk != 128 || Dv != 128 || Hk <= 0 || HV % Hk != 0 || rank <= 0 || rank > 256 || rank % 8 != 0 ||
        D % 8 != 0 || parity == nullptr)
        return VK_EINVAL;
    KdaChunkParams cp = {};
    cp.k = {(const __nv_bfloat16*)proj, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w_b, (const __nv_bfloat16*)w_fup,
            conv_w, A_log, dt_bias, (const __nv_bfloat16*)norm_w, (__nv_bfloat16*)conv, parity, conv_stride, S,
            (__nv_bfloat16*)out, nullptr, ldp, off_z, off_fd, D, Hk, HV, rank, eps};
    cp.accept = accept;
    cp.row_off = row_offset;
    cp.T = T;
    cp.write_state = write_state ? 1 : 0;
    static PerDeviceOnce once;
    VK_CUDA(once.run([] { return cudaFuncSetAttribute(kda_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(KdaChunkSmem)); }));
    return (int)vk_launch(kda_chunk_kernel, dim3(HV, B), dim3(512), sizeof(KdaChunkSmem), stream, cp);
}

int vk_kda_chunk(const void* proj, int ldp, int off_z, int off_fd, const void* h, const void* w_b, const void* w_fup,
                 const float* conv_w, const float* A_log, const float* dt_bias, const void* norm_w, void* conv,
                 const int* parity, size_t conv_stride, float* S, void* out, const int* accept, int write_state, int B, int T,
                 int D, int Hk, int HV, int Dk, int Dv, int rank, float eps, cudaStream_t stream) {
    return vk_kda_chunk_ragged(proj, ldp, off_z, off_fd, h, w_b, w_fup, conv_w, A_log, dt_bias, norm_w, conv, parity,
                               conv_stride, S, out, accept, nullptr, write_state, B, T, D, Hk, HV, Dk, Dv, rank, eps, stream);
}

int vk_kda_step(const void* proj, int ldp, int off_z, int off_fd, const void* h, const void* w_b, const void* w_fup,
                const float* conv_w, const float* A_log, const float* dt_bias, const void* norm_w, void* conv,
                const int* parity, size_t conv_stride, float* S, void* out, void* xrec_out, int B,
                int D, int Hk, int HV, int Dk, int Dv, int rank, float eps, cudaStream_t stream) {
    if (B <= 0 || Dk != 128 || Dv != 128 || Hk <= 0 || HV % Hk != 0 || rank <= 0 || rank > 256 || rank % 8 != 0 ||
        D % 8 != 0 || parity == nullptr || (xrec_out != nullptr && B > 16))
        return VK_EINVAL;
    KdaParams p = {(const __nv_bfloat16*)proj, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w_b,
                   (const __nv_bfloat16*)w_fup, conv_w, A_log, dt_bias, (const __nv_bfloat16*)norm_w,
                   (__nv_bfloat16*)conv, parity, conv_stride, S, (__nv_bfloat16*)out, (uint8_t*)xrec_out,
                   ldp, off_z, off_fd, D, Hk, HV, rank, eps};
    return (int)vk_launch(kda_step_kernel, dim3(HV, B), dim3(128), 0, stream, p);
}

}  // extern "C"
