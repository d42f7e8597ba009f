// Gated attention of the decode step over a paged, ragged KV cache: dense GQA and BCSA (local window + top-k far
// blocks, one joint softmax). Replaces Attention._batched / _bcsa_batched (volundr.py:737-791), the per-row index
// arithmetic of BCSAStep (batch.py:94-122), BatchBCSACache.write_ring / close_blocks (batch.py:224-259),
// BatchKVCache.attend (batch.py:306-316), _block_scores / _topk_blocks (volundr.py:601-618; kernels.py:8-98,
// 1168-1240) and the SDPA call (volundr.py:790).
//
// Layout. One page table [slot, max_pages] serves every attention layer: page i of a row holds its positions
// [64 i, 64 i + 64). Per layer: K, V pools bf16 [n_pages, KVH, 64, D] (post-norm, post-RoPE keys); pooled means of
// closed blocks of C positions PK, PV bf16 [n_pages, KVH, 64/C, D] (block j of a row sits in its page j C / 64, slot
// j mod 64/C); in indexer mode pooled indexer keys BK bf16 [n_pages, 64/C, Di] and the open block's keys
// IK [slot, C, Di]. The reference keeps a ring of the last W positions per row (slot p mod W); a page table holds the
// same positions without wrap-around and without padding rows to the longest one. Everything a step needs (slot,
// closing block, valid far blocks nv = max(0, (p - W + 1) / C), key counts) is derived on the GPU from pos[b].
//
// Modes (far, score): (pooled, indexer) is the reference: far keys are PK/PV rows picked by the shared indexer heads.
// (tokens, pooled_key) is the 64-token-block form: far keys are the tokens of the picked blocks, a block's score per
// kv head comes from that head's query heads against PK. Scores follow the reference's rounding chain
// bf16(bf16(mean_h fp32(bf16(q_h . k_j))) * scale) with the dot summed in a fixed order (4 consecutive elements per
// lane, then an xor tree), so the selected indices are reproducible bit for bit.
#include <atomic>

#include "common.cuh"
#include "xrec.cuh"

namespace {

constexpr int kPage = 64;
constexpr int kD = 128;  // head dim handled by these kernels

struct AttnGeom {
    int Hq, KVH, W, C, topk, IH, Di, NS;   // NS: selection groups (KVH in pooled_key mode, 1 in indexer mode, 0 dense)
    int far_tokens;                        // 1: far keys are tokens of the selected blocks; 0: pooled rows
    int max_pages;
};

// ------------------------------------------------------------------------------------------------ step bookkeeping
// For every row: allocate a page when the new token opens one (rows in order, so the assignment is deterministic),
// and write the step descriptor {pos, page id, row in page, closes block?, nv, nf, key count, window start}.
__global__ void batch_step_begin_kernel(const int* __restrict__ pos, int* __restrict__ table, int max_pages,
                                        int* __restrict__ free_list, int* __restrict__ free_top, int* __restrict__ desc,
                                        int B, int W, int C, int topk) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x != 0) return;
    int top = *free_top;
    for (int b = 0; b < B; b++) {
        const int p = pos[b];
        const int pi = p / kPage;
        if (pi >= max_pages) { vk_set_status(VK_ST_BAD_INDEX); continue; }
        if (p % kPage == 0) {
            if (top <= 0) { vk_set_status(VK_ST_POOL_EMPTY); continue; }
            table[b * max_pages + pi] = free_list[--top];
        }
        const int nv = W > 0 ? max(0, (p - W + 1) / C) : 0;
        const int nf = min(nv, topk);
        const int lo = W > 0 ? max(0, p - W + 1) : 0;
        int* d = desc + b * 8;
        d[0] = p; d[1] = table[b * max_pages + pi]; d[2] = p % kPage; d[3] = (W > 0 && (p + 1) % C == 0) ? 1 : 0;
        d[4] = nv; d[5] = nf; d[6] = (p - lo + 1) + nf; d[7] = lo;
    }
    *free_top = top;
}

// Pages for a chunk of tokens per row: row b is about to hold positions pos[b] .. pos[b] + lens[b] - 1; every position
// that starts a page takes one from the pool (rows in order, positions in order: the assignment is deterministic, and
// equals lens[b] single steps of batch_step_begin_kernel).
__global__ void pages_open_kernel(const int* __restrict__ pos, const int* __restrict__ lens, int* __restrict__ table,
                                  int max_pages, const int* __restrict__ free_list, int* __restrict__ free_top, int B) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x != 0) return;
    int top = *free_top;
    for (int b = 0; b < B; b++) {
        const int p0 = pos[b], p1 = p0 + lens[b];
        for (int pi = (p0 + kPage - 1) / kPage; pi * kPage < p1; pi++) {
            if (pi >= max_pages) { vk_set_status(VK_ST_BAD_INDEX); break; }
            if (top <= 0) { vk_set_status(VK_ST_POOL_EMPTY); break; }
            table[b * max_pages + pi] = free_list[--top];
        }
    }
    *free_top = top;
}

// Pages go back to the pool: for item i, the table entries [first[i], last[i]) of row rows[i] (entries that hold no
// page are skipped), pushed in ascending order, or descending with `reverse` (a row that leaves hands its pages back
// last first, so that the next row to grow takes them in the order the old row did); the entries become -1.
__global__ void pages_release_kernel(const int* __restrict__ rows, const int* __restrict__ first, const int* __restrict__ last,
                                     int n, int reverse, int* __restrict__ table, int max_pages, int* __restrict__ free_list,
                                     int* __restrict__ free_top, int n_pages) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x != 0) return;
    int top = *free_top;
    for (int i = 0; i < n; i++) {
        const int b = rows[i];
        const int a = max(first[i], 0), z = min(last[i], max_pages);
        for (int k = 0; k < z - a; k++) {
            const int pi = reverse ? z - 1 - k : a + k;
            const int page = table[b * max_pages + pi];
            if (page < 0) continue;
            if (page >= n_pages || top >= n_pages) { vk_set_status(VK_ST_BAD_INDEX); continue; }
            free_list[top++] = page;
            table[b * max_pages + pi] = -1;
        }
    }
    *free_top = top;
}
// every row holds one more token; the KDA conv-state buffers swap roles
__global__ void batch_step_end_kernel(int* pos, int* parity, int B) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B) pos[b] += 1;
    if (b == 0 && parity != nullptr) *parity ^= 1;
}

// ------------------------------------------------------------------------------------------------ projections -> cache
struct PrepParams {
    const __nv_bfloat16* proj;    // [B, ldp]: per q head [q (D) | gate (D)], then k [KVH, D] at off_k, v at off_v
    const __nv_bfloat16* idxq;    // [B, IH*Di] or null
    const __nv_bfloat16* idxk;    // [B, Di] or null
    const __nv_bfloat16* q_norm;  // [D] offset-norm weights
    const __nv_bfloat16* k_norm;
    const __nv_bfloat16* idx_norm;  // [Di]
    const int* pos;               // [B]
    const int* table;             // [slots, max_pages]
    __nv_bfloat16* q;             // [B, Hq, D]
    __nv_bfloat16* qi;            // [B, IH, Di]
    __nv_bfloat16 *K, *V, *PK, *PV, *BK, *IK;
    int ldp, off_k, off_v, n_pages, rope_dims;
    double log2_theta;
    float eps;
    AttnGeom g;
    int mode;                     // 0: write the row and pool the block it closes; 1: write only; 2: pool only
    const int* row_map;           // null, or [B]: the cache row whose open-block indexer keys (IK) row b uses
    // Rows that are consecutive positions of one sequence (modes 1 and 2): the normed indexer key of row b goes to
    // ikc[b] (the C-slot ring of the cache row cannot hold more than one open block), and a block that closes inside
    // the chunk is pooled from the chunk's own keys, plus the ring for the positions in front of first_pos[b], the
    // first position the chunk brought for this row's sequence. The ring itself is left alone.
    __nv_bfloat16* ikc;           // null, or [B, Di]
    const int* first_pos;         // [B] (with ikc)
};

// offset RMSNorm of one 128-vector held 4 elements per lane; returns bf16-rounded values
__device__ __forceinline__ void head_norm128(float (&x)[4], const __nv_bfloat16* w, int lane, float eps) {
    float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss * (1.f / 128.f) + eps);
#pragma unroll
    for (int e = 0; e < 4; e++) x[e] = bfr((x[e] * inv) * (1.f + bf2f(w[4 * lane + e])));
}

__device__ __forceinline__ void load4(const __nv_bfloat16* p, int lane, float (&x)[4]) {
    const uint2 u = *reinterpret_cast<const uint2*>(p + 4 * lane);
    x[0] = bf_lo(u.x); x[1] = bf_hi(u.x); x[2] = bf_lo(u.y); x[3] = bf_hi(u.y);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, int lane, const float (&x)[4]) {
    uint2 u;
    u.x = pack_bf2(x[0], x[1]);
    u.y = pack_bf2(x[2], x[3]);
    *reinterpret_cast<uint2*>(p + 4 * lane) = u;
}

// NeoX rotate-half on the first rd dims of a 128-vector spread 4 per lane; cs / sn [rd / 2] hold cos / sin of
// angle_i = pos * theta^(-2i/rd), computed in double (rope_table).
__device__ __forceinline__ void rope128(float (&x)[4], int lane, int rd, const double* cs, const double* sn) {
    const int half = rd / 2;
    float other[4];
    // partner lane holds the element half a rotation away
    const int shift = half / 4;  // lanes per half (rd a multiple of 8)
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const float up = __shfl_down_sync(0xffffffffu, x[e], shift);
        const float dn = __shfl_up_sync(0xffffffffu, x[e], shift);
        other[e] = (4 * lane < half) ? up : dn;
    }
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const int d = 4 * lane + e;
        if (d < rd) {
            const int i = d < half ? d : d - half;
            const double v = d < half ? (double)x[e] * cs[i] - (double)other[e] * sn[i] : (double)x[e] * cs[i] + (double)other[e] * sn[i];
            x[e] = bfr((float)v);
        }
    }
}

// Mean of the C rows of a closed block, added in order in fp32, times 1/C, rounded once (BCSACache._pool,
// volundr.py:470-476). Each lane reads the four elements it also wrote for the newest row, so the warp that wrote that
// row can pool right away.
__device__ __forceinline__ void pool_rows(const __nv_bfloat16* src, int C, int lane, __nv_bfloat16* dst) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int i0 = 0; i0 < C; i0 += 8) {
        float x[8][4];
#pragma unroll
        for (int u = 0; u < 8; u++)
            if (i0 + u < C) load4(src + (size_t)(i0 + u) * kD, lane, x[u]);
#pragma unroll
        for (int u = 0; u < 8; u++) {
            if (i0 + u < C) {
#pragma unroll
                for (int e = 0; e < 4; e++) acc[e] += x[u][e];
            }
        }
    }
    const float invc = 1.f / (float)C;
#pragma unroll
    for (int e = 0; e < 4; e++) acc[e] = bfr(acc[e] * invc);
    store4(dst, lane, acc);
}

// One warp per head: grid (rows, ceil(heads / 8)). The warp that writes a row's K (V, indexer key) also forms the
// pooled mean of the block when this position closes one.
__global__ void __launch_bounds__(256) attn_prep_kernel(const PrepParams p) {
    __shared__ double cs_sm[64], sn_sm[64];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const AttnGeom& g = p.g;
    const int pos = p.pos[b];
    const int page = p.table[b * g.max_pages + pos / kPage];
    const int row = pos % kPage;
    if (page < 0 || page >= p.n_pages) {
        if (threadIdx.x == 0 && blockIdx.y == 0) vk_set_status(VK_ST_BAD_INDEX);
        return;
    }
    const int hd0 = blockIdx.y * 8;
    if (hd0 < g.Hq + g.KVH && threadIdx.x < p.rope_dims / 2) {   // this CTA has heads that rotate
        const int i = threadIdx.x;
        const double ang = (double)pos * exp2(-(2.0 * i / p.rope_dims) * p.log2_theta);
        double sn, cs;
        sincos(ang, &sn, &cs);
        cs_sm[i] = cs;
        sn_sm[i] = sn;
    }
    __syncthreads();
    const __nv_bfloat16* pr = p.proj + (size_t)b * p.ldp;
    const int nheads = g.Hq + 2 * g.KVH + (p.idxq ? g.IH + 1 : 0);
    const int hd = hd0 + warp;
    if (hd >= nheads) return;
    const bool wr = p.mode != 2;                                          // write this position's rows
    const bool closes = p.mode != 1 && g.W > 0 && (pos + 1) % g.C == 0;   // pool the block this position closes
    const int slot = (pos / g.C) % (kPage / g.C);
    const int r0 = row - (g.C - 1);
    float x[4];
    if (hd < g.Hq) {                                   // query head: norm, rope
        if (!wr) return;
        load4(pr + (size_t)hd * 2 * kD, lane, x);
        head_norm128(x, p.q_norm, lane, p.eps);
        rope128(x, lane, p.rope_dims, cs_sm, sn_sm);
        store4(p.q + ((size_t)b * g.Hq + hd) * kD, lane, x);
    } else if (hd < g.Hq + g.KVH) {                    // key head: norm, rope, into the page
        const int kv = hd - g.Hq;
        __nv_bfloat16* Kp = p.K + ((size_t)page * g.KVH + kv) * kPage * kD;
        if (wr) {
            load4(pr + p.off_k + (size_t)kv * kD, lane, x);
            head_norm128(x, p.k_norm, lane, p.eps);
            rope128(x, lane, p.rope_dims, cs_sm, sn_sm);
            store4(Kp + (size_t)row * kD, lane, x);
        }
        if (closes) pool_rows(Kp + (size_t)r0 * kD, g.C, lane, p.PK + (((size_t)page * g.KVH + kv) * (kPage / g.C) + slot) * kD);
    } else if (hd < g.Hq + 2 * g.KVH) {                // value head: as projected
        const int kv = hd - g.Hq - g.KVH;
        __nv_bfloat16* Vp = p.V + ((size_t)page * g.KVH + kv) * kPage * kD;
        if (wr) {
            load4(pr + p.off_v + (size_t)kv * kD, lane, x);
            store4(Vp + (size_t)row * kD, lane, x);
        }
        if (closes) pool_rows(Vp + (size_t)r0 * kD, g.C, lane, p.PV + (((size_t)page * g.KVH + kv) * (kPage / g.C) + slot) * kD);
    } else if (hd < g.Hq + 2 * g.KVH + g.IH) {         // indexer query heads
        if (!wr) return;
        const int ih = hd - g.Hq - 2 * g.KVH;
        load4(p.idxq + ((size_t)b * g.IH + ih) * kD, lane, x);
        head_norm128(x, p.idx_norm, lane, p.eps);
        store4(p.qi + ((size_t)b * g.IH + ih) * kD, lane, x);
    } else {                                           // indexer key of this position -> open block slot
        const int ikrow = p.row_map != nullptr ? p.row_map[b] : b;
        __nv_bfloat16* Ip = p.IK + (size_t)ikrow * g.C * kD;
        if (wr) {
            load4(p.idxk + (size_t)b * kD, lane, x);
            head_norm128(x, p.idx_norm, lane, p.eps);
            store4(p.ikc != nullptr ? p.ikc + (size_t)b * kD : Ip + (size_t)(pos % g.C) * kD, lane, x);
        }
        if (closes) {
            __nv_bfloat16* dst = p.BK + ((size_t)page * (kPage / g.C) + slot) * kD;
            if (p.ikc == nullptr) {
                pool_rows(Ip, g.C, lane, dst);
            } else {   // positions pos - C + 1 .. pos in order: from the chunk's rows, or from the ring in front of it
                const int first = p.first_pos[b];
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                for (int i = 0; i < g.C; i++) {
                    const int tp = pos - (g.C - 1) + i;
                    const __nv_bfloat16* src = tp >= first ? p.ikc + (size_t)(b - (pos - tp)) * kD : Ip + (size_t)(tp % g.C) * kD;
                    float y[4];
                    load4(src, lane, y);
#pragma unroll
                    for (int e = 0; e < 4; e++) acc[e] += y[e];
                }
                const float invc = 1.f / (float)g.C;
#pragma unroll
                for (int e = 0; e < 4; e++) acc[e] = bfr(acc[e] * invc);
                store4(dst, lane, acc);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------ far-block selection
struct SelectParams {
    const __nv_bfloat16* q;       // score queries: qi [B, IH, Di] (indexer) or q [B, Hq, D] (pooled_key)
    const __nv_bfloat16* keys;    // BK [n_pages, 64/C, Di] (indexer) or PK [n_pages, KVH, 64/C, D] (pooled_key)
    const int* pos;
    const int* table;
    uint32_t* scratch;            // [B, NS, cap] sort keys
    int* sel;                     // [B, NS, topk] ascending block indices, -1 padded
    int* nsel;                    // [B, NS]
    int cap, n_pages;
    float scale;                  // Di^-1/2
    AttnGeom g;
};

constexpr int kFastBlocks = 512;     // blocks per (row, group) the shared-memory path of the selection holds
constexpr int kKeyStride = 272;      // bytes between key rows in shared memory (256 + 16: conflict-free 16-byte reads)
constexpr size_t kSelectSmem = (size_t)kFastBlocks * kKeyStride + 8 * 128 * 4 + kFastBlocks * 4;

__device__ __forceinline__ uint32_t score_key(float s, int j) {
    const uint32_t u = __float_as_uint(s) >> 16;  // s is bf16-valued
    const uint32_t mono = (u & 0x8000u) ? (0xFFFFu - u) : (u | 0x8000u);
    return (mono << 16) | (0xFFFFu - (uint32_t)j);
}

__global__ void __launch_bounds__(256) bcsa_select_kernel(const SelectParams p) {
    __shared__ int hist[256];
    __shared__ uint32_t s_prefix;
    __shared__ int s_k;
    __shared__ int wcount[8];
    __shared__ int s_base;
    pdl_launch_dependents();
    pdl_wait();
    const AttnGeom& g = p.g;
    const int ns = blockIdx.x, b = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = p.pos[b];
    const int nv = max(0, (pos - g.W + 1) / g.C);
    int* sel = p.sel + ((size_t)b * g.NS + ns) * g.topk;
    if (nv <= g.topk) {
        for (int i = threadIdx.x; i < g.topk; i += 256) sel[i] = i < nv ? i : -1;
        if (threadIdx.x == 0) p.nsel[b * g.NS + ns] = nv;
        return;
    }
    if (nv > p.cap || nv > 65536 || nv > g.max_pages * (kPage / g.C)) {
        if (threadIdx.x == 0) { vk_set_status(VK_ST_BAD_INDEX); p.nsel[b * g.NS + ns] = 0; }
        return;
    }
    const bool per_kv = g.NS > 1;
    const int nh = per_kv ? g.Hq / g.KVH : g.IH;
    const __nv_bfloat16* qb = per_kv ? p.q + ((size_t)b * g.Hq + (size_t)ns * nh) * kD : p.q + (size_t)b * g.IH * kD;
    const int spp = kPage / g.C;  // pooled slots per page
    if (nv <= kFastBlocks) {
        // ---- up to 512 blocks (32K tokens at C = 64): everything in shared memory. All key rows are fetched at once
        // (one round of memory latency instead of one per pass), every thread scores whole blocks, and the k-th
        // largest key is found by counting. The arithmetic is that of the general path below, addition by addition:
        // the 32 four-element partial sums of a dot product are combined in the order of the warp's xor tree.
        extern __shared__ __align__(16) uint8_t dsm[];
        uint8_t* krows = dsm;                                                    // [nv][272 bytes]
        float* qsm = reinterpret_cast<float*>(dsm + (size_t)kFastBlocks * kKeyStride);   // [8][128]
        uint32_t* skeys = reinterpret_cast<uint32_t*>(qsm + 8 * kD);             // [512]
        // (the pages of all blocks first, in one round of loads: a table load in front of every copy below would
        // serialise them, the copy instructions being ordered against memory operations)
        int bad = 0;
        for (int j = threadIdx.x; j < nv; j += 256) {
            const int page = p.table[b * g.max_pages + (j / spp)];
            bad |= (page < 0 || page >= p.n_pages);
            skeys[j] = (uint32_t)page;
        }
        if (__syncthreads_or(bad)) {   // a page number outside the pool: nothing is fetched through it
            if (threadIdx.x == 0) { vk_set_status(VK_ST_BAD_INDEX); p.nsel[b * g.NS + ns] = 0; }
            return;
        }
        for (int idx = threadIdx.x; idx < nv * 16; idx += 256) {
            const int j = idx >> 4, piece = idx & 15;
            const int page = (int)skeys[j];
            const __nv_bfloat16* kr = per_kv ? p.keys + (((size_t)page * g.KVH + ns) * spp + j % spp) * kD
                                             : p.keys + ((size_t)page * spp + j % spp) * kD;
            cp_async16(krows + (size_t)j * kKeyStride + piece * 16, reinterpret_cast<const uint8_t*>(kr) + piece * 16);
        }
        cp_async_commit();
        for (int i = threadIdx.x; i < nh * kD; i += 256) qsm[i] = bf2f(qb[i]);
        const int nv4 = (nv + 3) >> 2;
        cp_async_wait0();
        __syncthreads();   // (also: every thread is done with the page numbers held in skeys)
        for (int i = nv + threadIdx.x; i < nv4 * 4; i += 256) skeys[i] = 0u;   // below every real key
        const float inv_nh = 1.f / (float)nh;
        for (int j = threadIdx.x; j < nv; j += 256) {
            const uint8_t* kr = krows + (size_t)j * kKeyStride;
            float sc = 0.f;
#pragma unroll 1
            for (int h = 0; h < nh; h++) {
                const float4* qh = reinterpret_cast<const float4*>(qsm + h * kD);
                float s1[16];   // s1[l] = partial of "lane" l + partial of "lane" l + 16
#pragma unroll
                for (int m = 0; m < 8; m++) {
                    const uint4 ka = *reinterpret_cast<const uint4*>(kr + m * 16);         // elements 8m .. 8m+7
                    const uint4 kb = *reinterpret_cast<const uint4*>(kr + 128 + m * 16);   // elements 64+8m .. 64+8m+7
                    const float4 q0 = qh[2 * m], q1 = qh[2 * m + 1], q2 = qh[16 + 2 * m], q3 = qh[17 + 2 * m];
                    float a0 = q0.x * bf_lo(ka.x); a0 = fmaf(q0.y, bf_hi(ka.x), a0); a0 = fmaf(q0.z, bf_lo(ka.y), a0); a0 = fmaf(q0.w, bf_hi(ka.y), a0);
                    float a1 = q1.x * bf_lo(ka.z); a1 = fmaf(q1.y, bf_hi(ka.z), a1); a1 = fmaf(q1.z, bf_lo(ka.w), a1); a1 = fmaf(q1.w, bf_hi(ka.w), a1);
                    float c0 = q2.x * bf_lo(kb.x); c0 = fmaf(q2.y, bf_hi(kb.x), c0); c0 = fmaf(q2.z, bf_lo(kb.y), c0); c0 = fmaf(q2.w, bf_hi(kb.y), c0);
                    float c1 = q3.x * bf_lo(kb.z); c1 = fmaf(q3.y, bf_hi(kb.z), c1); c1 = fmaf(q3.z, bf_lo(kb.w), c1); c1 = fmaf(q3.w, bf_hi(kb.w), c1);
                    s1[2 * m] = a0 + c0;
                    s1[2 * m + 1] = a1 + c1;
                }
#pragma unroll
                for (int l = 0; l < 8; l++) s1[l] += s1[l + 8];
#pragma unroll
                for (int l = 0; l < 4; l++) s1[l] += s1[l + 4];
                s1[0] += s1[2]; s1[1] += s1[3];
                sc += bfr(s1[0] + s1[1]);
            }
            sc = bfr(sc * inv_nh);
            sc = bfr(sc * p.scale);
            skeys[j] = score_key(sc, j);
        }
        __syncthreads();
        if (threadIdx.x == 0) s_base = 0;
        __syncthreads();
        for (int j0 = 0; j0 < nv; j0 += 256) {
            const int j = j0 + threadIdx.x;
            bool take = false;
            if (j < nv) {
                const uint32_t my = skeys[j];
                int above = 0;
                for (int i = 0; i < nv4; i++) {
                    const uint4 v = reinterpret_cast<const uint4*>(skeys)[i];
                    above += (v.x > my) + (v.y > my) + (v.z > my) + (v.w > my);
                }
                take = above < g.topk;
            }
            const uint32_t bal = __ballot_sync(0xffffffffu, take);
            if (lane == 0) wcount[warp] = __popc(bal);
            __syncthreads();
            int off = s_base;
            for (int w = 0; w < warp; w++) off += wcount[w];
            if (take) {
                const int r = off + __popc(bal & ((1u << lane) - 1u));
                if (r < g.topk) sel[r] = j;
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                int t = 0;
                for (int w = 0; w < 8; w++) t += wcount[w];
                s_base += t;
            }
            __syncthreads();
        }
        if (threadIdx.x == 0) p.nsel[b * g.NS + ns] = g.topk;
        return;
    }
    uint32_t* keys = p.scratch + ((size_t)b * g.NS + ns) * p.cap;
    float qv[8][4];  // fully unrolled below, so the heads stay in registers
#pragma unroll
    for (int h = 0; h < 8; h++) {
        if (h < nh) load4(qb + (size_t)h * kD, lane, qv[h]);
        else { qv[h][0] = qv[h][1] = qv[h][2] = qv[h][3] = 0.f; }
    }
    const float inv_nh = 1.f / (float)nh;
    // four blocks per warp and pass: their table entries and keys are fetched together, then scored one by one
    for (int j0 = warp * 4; j0 < nv; j0 += 32) {
        float kx[4][4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int j = j0 + u;
            kx[u][0] = kx[u][1] = kx[u][2] = kx[u][3] = 0.f;
            if (j < nv) {
                const int page = p.table[b * g.max_pages + (j / spp)];
                if (page < 0 || page >= p.n_pages) {   // outside the pool: scored as zeros, reported
                    if (lane == 0) vk_set_status(VK_ST_BAD_INDEX);
                } else {
                    const __nv_bfloat16* kr = per_kv ? p.keys + (((size_t)page * g.KVH + ns) * spp + j % spp) * kD
                                                     : p.keys + ((size_t)page * spp + j % spp) * kD;
                    load4(kr, lane, kx[u]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int j = j0 + u;
            if (j >= nv) break;
            float sc = 0.f;
#pragma unroll
            for (int h = 0; h < 8; h++) {
                if (h >= nh) break;
                float a = qv[h][0] * kx[u][0];
                a = fmaf(qv[h][1], kx[u][1], a);
                a = fmaf(qv[h][2], kx[u][2], a);
                a = fmaf(qv[h][3], kx[u][3], a);
                a = warp_sum(a);
                sc += bfr(a);
            }
            sc = bfr(sc * inv_nh);
            sc = bfr(sc * p.scale);
            if (lane == 0) keys[j] = score_key(sc, j);
        }
    }
    __syncthreads();
    // ---- radix select: the topk-th largest key (keys are unique), 8 bits per pass from the top
    if (threadIdx.x == 0) { s_prefix = 0; s_k = g.topk; }
    uint32_t mask = 0;
    for (int pass = 3; pass >= 0; pass--) {
        const int shift = 8 * pass;
        hist[threadIdx.x] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        for (int j = threadIdx.x; j < nv; j += 256) {
            const uint32_t k = __ldcg(keys + j);
            if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 0xFF], 1);
        }
        __syncthreads();
        if (warp == 0) {
            // the digit d with count(digits > d) < need <= count(digits >= d): lane l holds digits 8l .. 8l+7
            int c8[8], mine = 0;
#pragma unroll
            for (int e = 0; e < 8; e++) { c8[e] = hist[lane * 8 + e]; mine += c8[e]; }
            int incl = mine;  // keys in the digits of this lane and of every higher lane
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_down_sync(0xffffffffu, incl, o);
                if (lane + o < 32) incl += v;
            }
            const int suffix = incl - mine;
            const int need = s_k;
            const bool here = suffix < need && suffix + mine >= need;
            if (here) {
                int acc = suffix, d = lane * 8 + 7;
                for (int e = 7; e >= 0; e--) {
                    if (acc + c8[e] >= need) { d = lane * 8 + e; break; }
                    acc += c8[e];
                }
                s_k = need - acc;
                s_prefix = prefix | ((uint32_t)d << shift);
            }
        }
        mask |= 0xFFu << shift;
        __syncthreads();
    }
    const uint32_t thr = s_prefix;
    // ---- ordered compaction: indices of keys >= thr, ascending
    if (threadIdx.x == 0) s_base = 0;
    __syncthreads();
    for (int j0 = 0; j0 < nv; j0 += 256) {
        const int j = j0 + threadIdx.x;
        const bool take = j < nv && __ldcg(keys + j) >= thr;
        const uint32_t bal = __ballot_sync(0xffffffffu, take);
        if (lane == 0) wcount[warp] = __popc(bal);
        __syncthreads();
        int off = s_base;
        for (int w = 0; w < warp; w++) off += wcount[w];
        if (take) {
            const int r = off + __popc(bal & ((1u << lane) - 1u));
            if (r < g.topk) sel[r] = j;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int t = 0;
            for (int w = 0; w < 8; w++) t += wcount[w];
            s_base += t;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) p.nsel[b * g.NS + ns] = g.topk;
}

// ------------------------------------------------------------------------------------------------ attention
struct AttendParams {
    const __nv_bfloat16* q;     // [B, Hq, D]
    const __nv_bfloat16 *K, *V, *PK, *PV;
    const int* pos;
    const int* table;
    const int* sel;             // [B, NS, topk] or null
    const int* nsel;
    float* part;                // [B, KVH, nsplit, G, D + 2]: O (D), m, l
    int nsplit, n_pages;
    float scale;
    AttnGeom g;
};

constexpr int kRowStride = kD + 8;  // bf16 elements; keeps 16-byte row reads conflict-free

// A page number read from a row's table, checked against the pool: an entry outside it is reported through the
// status word and replaced by page 0, so nothing is ever read or written outside the pool.
__device__ __forceinline__ int checked_page(int page, int n_pages) {
    if (page < 0 || page >= n_pages) {
        vk_set_status(VK_ST_BAD_INDEX);
        return 0;
    }
    return page;
}

template <int G>
__global__ void __launch_bounds__(128) attend_decode_kernel(const AttendParams p) {
    __shared__ __align__(16) __nv_bfloat16 Ks[kPage * kRowStride];
    __shared__ __align__(16) __nv_bfloat16 Vs[kPage * kRowStride];
    __shared__ __align__(16) float qs[G * kD];
    __shared__ float sc[G * kPage];
    __shared__ float umax[G], usum[G];
    __shared__ const __nv_bfloat16* rowK[kPage];
    __shared__ const __nv_bfloat16* rowV[kPage];
    pdl_launch_dependents();
    pdl_wait();
    const AttnGeom& g = p.g;
    const int split = blockIdx.x, kv = blockIdx.y, b = blockIdx.z;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int pos = p.pos[b];
    const int lo = g.W > 0 ? max(0, pos - g.W + 1) : 0;
    const int wp0 = lo / kPage, nwp = pos / kPage - wp0 + 1;
    const int ns = g.NS > 1 ? kv : 0;
    const int nf = (p.sel != nullptr && g.NS > 0) ? p.nsel[b * g.NS + ns] : 0;
    const int* sel = p.sel ? p.sel + ((size_t)b * g.NS + ns) * g.topk : nullptr;
    const int spp = g.W > 0 ? kPage / g.C : 1;
    const int nfu = g.far_tokens ? nf : (nf + kPage - 1) / kPage;  // far units
    const int U = nwp + nfu;

    for (int i = t; i < G * kD; i += 128) qs[i] = bf2f(p.q[((size_t)b * g.Hq + (size_t)kv * G) * kD + i]) * p.scale;
    float m_run[G], l_run[G], O[G];
#pragma unroll
    for (int h = 0; h < G; h++) { m_run[h] = -INFINITY; l_run[h] = 0.f; O[h] = 0.f; }

    for (int u = split; u < U; u += p.nsplit) {
        __syncthreads();
        // ---- which rows make up this unit
        int nrows;
        if (u < nwp) {
            const int page = checked_page(p.table[b * g.max_pages + wp0 + u], p.n_pages);
            const int ra = u == 0 ? lo % kPage : 0;
            const int rb = u == nwp - 1 ? pos % kPage : kPage - 1;
            nrows = rb - ra + 1;
            if (t < nrows) {
                const size_t off = (((size_t)page * g.KVH + kv) * kPage + ra + t) * kD;
                rowK[t] = p.K + off;
                rowV[t] = p.V + off;
            }
        } else if (g.far_tokens) {
            const int j = sel[u - nwp];
            const int tok0 = j * g.C;
            const int page = checked_page(p.table[b * g.max_pages + tok0 / kPage], p.n_pages);
            nrows = g.C;
            if (t < nrows) {
                const size_t off = (((size_t)page * g.KVH + kv) * kPage + tok0 % kPage + t) * kD;
                rowK[t] = p.K + off;
                rowV[t] = p.V + off;
            }
        } else {
            const int f0 = (u - nwp) * kPage;
            nrows = min(kPage, nf - f0);
            if (t < nrows) {
                const int j = sel[f0 + t];
                const int page = checked_page(p.table[b * g.max_pages + (j / spp)], p.n_pages);
                const size_t off = (((size_t)page * g.KVH + kv) * spp + j % spp) * kD;
                rowK[t] = p.PK + off;
                rowV[t] = p.PV + off;
            }
        }
        __syncthreads();
        // ---- stage the rows: 16-byte asynchronous copies, all in flight at once (16 per 256-byte row)
        for (int i = t; i < nrows * 16; i += 128) {
            const int r = i >> 4, cch = i & 15;
            cp_async16(Ks + r * kRowStride + cch * 8, rowK[r] + cch * 8);
            cp_async16(Vs + r * kRowStride + cch * 8, rowV[r] + cch * 8);
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();
        // ---- scores: thread (key i = t % 64, heads h = t / 64, t / 64 + 2, ...)
        {
            const int i = t & 63;
            for (int h = t >> 6; h < G; h += 2) {
                float a = -INFINITY;
                if (i < nrows) {
                    a = 0.f;
                    const __nv_bfloat16* kr = Ks + i * kRowStride;
                    const float* qh = qs + h * kD;
#pragma unroll 4
                    for (int d = 0; d < kD; d += 8) {
                        const uint4 kk = *reinterpret_cast<const uint4*>(kr + d);
                        a = fmaf(bf_lo(kk.x), qh[d], a); a = fmaf(bf_hi(kk.x), qh[d + 1], a);
                        a = fmaf(bf_lo(kk.y), qh[d + 2], a); a = fmaf(bf_hi(kk.y), qh[d + 3], a);
                        a = fmaf(bf_lo(kk.z), qh[d + 4], a); a = fmaf(bf_hi(kk.z), qh[d + 5], a);
                        a = fmaf(bf_lo(kk.w), qh[d + 6], a); a = fmaf(bf_hi(kk.w), qh[d + 7], a);
                    }
                }
                sc[h * kPage + i] = a;
            }
        }
        __syncthreads();
        // ---- softmax pieces of this unit per head (warp w takes heads w, w + 4, ...): max, exp, sum
        for (int h = warp; h < G; h += 4) {
            const float s0 = sc[h * kPage + lane], s1 = sc[h * kPage + 32 + lane];
            const float mx = warp_max(fmaxf(s0, s1));  // finite: a unit has at least one row
            const float p0 = __expf(s0 - mx), p1 = __expf(s1 - mx);
            sc[h * kPage + lane] = p0;
            sc[h * kPage + 32 + lane] = p1;
            const float sum = warp_sum(p0 + p1);
            if (lane == 0) { umax[h] = mx; usum[h] = sum; }
        }
        __syncthreads();
        // every thread keeps the running max / sum of every head (identical values in all threads)
        float w_unit[G];
#pragma unroll
        for (int h = 0; h < G; h++) {
            const float mx = umax[h];
            const float m_new = fmaxf(m_run[h], mx);
            const float a_old = m_run[h] == -INFINITY ? 0.f : __expf(m_run[h] - m_new);
            const float a_new = __expf(mx - m_new);
            l_run[h] = l_run[h] * a_old + usum[h] * a_new;
            O[h] *= a_old;
            w_unit[h] = a_new;
            m_run[h] = m_new;
        }
        // ---- O[h][d = t] += sum_i p[h][i] V[i][t]
        for (int i = 0; i < nrows; i++) {
            const float v = bf2f(Vs[i * kRowStride + t]);
#pragma unroll
            for (int h = 0; h < G; h++) O[h] = fmaf(sc[h * kPage + i] * w_unit[h], v, O[h]);
        }
    }
    float* out = p.part + (((size_t)b * g.KVH + kv) * p.nsplit + split) * G * (kD + 2);
#pragma unroll
    for (int h = 0; h < G; h++) {
        out[h * (kD + 2) + t] = O[h];
        if (t == 0) { out[h * (kD + 2) + kD] = m_run[h]; out[h * (kD + 2) + kD + 1] = l_run[h]; }
    }
}

// merge the splits of one query head, divide, round, apply sigmoid(gate) (volundr.py:177-179, :752-753)
__global__ void __launch_bounds__(128) attend_merge_kernel(const float* __restrict__ part, const __nv_bfloat16* __restrict__ proj,
                                                           int ldp, __nv_bfloat16* __restrict__ out, uint8_t* __restrict__ xrec_out,
                                                           int Hq, int KVH, int nsplit) {
    __shared__ float red[4];
    pdl_launch_dependents();
    pdl_wait();
    const int hq = blockIdx.x, b = blockIdx.y, t = threadIdx.x;
    const int G = Hq / KVH, kv = hq / G, h = hq % G;
    const float* base = part + (((size_t)b * KVH + kv) * nsplit) * G * (kD + 2) + (size_t)h * (kD + 2);
    // (loads in batches of eight independent ones: the splits' partial results sit in L2, and a loop of dependent
    // loads would pay that latency once per split)
    const size_t sstride = (size_t)G * (kD + 2);
    float m = -INFINITY;
    for (int s0 = 0; s0 < nsplit; s0 += 8) {
        float mv[8];
#pragma unroll
        for (int u = 0; u < 8; u++) mv[u] = s0 + u < nsplit ? base[(size_t)(s0 + u) * sstride + kD] : -INFINITY;
#pragma unroll
        for (int u = 0; u < 8; u++) m = fmaxf(m, mv[u]);
    }
    float l = 0.f, o = 0.f;
    for (int s0 = 0; s0 < nsplit; s0 += 8) {
        float mv[8], lv[8], ov8[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const bool in = s0 + u < nsplit;
            const float* ps = base + (size_t)(in ? s0 + u : 0) * sstride;
            mv[u] = in ? ps[kD] : -INFINITY;
            lv[u] = ps[kD + 1];
            ov8[u] = ps[t];
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
            if (mv[u] != -INFINITY) {   // (an empty split holds no sums)
                const float w = __expf(mv[u] - m);
                l = fmaf(lv[u], w, l);
                o = fmaf(ov8[u], w, o);
            }
        }
    }
    const float ob = bfr(o / l);
    const float gate = bf2f(proj[(size_t)b * ldp + (size_t)hq * 2 * kD + kD + t]);
    const float ov = bfr(ob * (1.f / (1.f + expf(-gate))));
    out[((size_t)b * Hq + hq) * kD + t] = f2bf(ov);
    if (xrec_out != nullptr) {
        const int kg = hq * 2 + (t >> 6);
        *xrec_elem(xrec_out, kg, b, t & 63) = f2bf(ov);
        const float ws = warp_sum(ov);
        if ((t & 31) == 0) red[t >> 5] = ws;
        __syncthreads();
        if ((t & 63) == 0) xrec_store_sum(xrec_out, kg, b, red[t >> 5] + red[(t >> 5) + 1]);
    }
}

// ------------------------------------------------------------------------------------------------ attention, tensor cores
// The same split-KV decode attention with both products on the tensor cores: S = Q K^T with the G query heads of the
// kv head as the 16-row A operand (rows >= G zero) and P V with bf16 probabilities. Per unit of up to 64 keys:
// 4 warps x (16 keys) for S, softmax pieces per head, 4 warps x (32 dims) for O. fp32 running max / sum / O.
constexpr int kPStride = kPage + 8;   // bf16 elements per row of the probability tile

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int G>
__global__ void __launch_bounds__(128) attend_decode_tc_kernel(const AttendParams p) {
    __shared__ __align__(16) __nv_bfloat16 Ks[kPage * kRowStride];
    __shared__ __align__(16) __nv_bfloat16 Vs[kPage * kRowStride];
    __shared__ __align__(16) __nv_bfloat16 Qs[16 * kRowStride];
    __shared__ __align__(16) __nv_bfloat16 Ps[16 * kPStride];
    __shared__ __align__(16) float sc[8 * kPage];
    __shared__ float s_aold[8], s_m[8], s_l[8];
    __shared__ const __nv_bfloat16* rowK[2][kPage];
    __shared__ const __nv_bfloat16* rowV[2][kPage];
    pdl_launch_dependents();
    pdl_wait();
#if defined(VK_TRACE) && VK_TRACE == 7
    long long tr[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const long long tr_start = clock64();
#define AT_T(var) const long long var = clock64()
#define AT_ACC(slot, a, b) tr[slot] += (b) - (a)
#else
#define AT_T(var) do { } while (0)
#define AT_ACC(slot, a, b) do { } while (0)
#endif
    const AttnGeom& g = p.g;
    const int split = blockIdx.x, kv = blockIdx.y, b = blockIdx.z;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int gq = lane >> 2, tq = lane & 3;
    const int pos = p.pos[b];
    const int lo = g.W > 0 ? max(0, pos - g.W + 1) : 0;
    const int wp0 = lo / kPage, nwp = pos / kPage - wp0 + 1;
    const int ns = g.NS > 1 ? kv : 0;
    const int nf = (p.sel != nullptr && g.NS > 0) ? p.nsel[b * g.NS + ns] : 0;
    const int* sel = p.sel ? p.sel + ((size_t)b * g.NS + ns) * g.topk : nullptr;
    const int spp = g.W > 0 ? kPage / g.C : 1;
    const int nfu = g.far_tokens ? nf : (nf + kPage - 1) / kPage;
    const int U = nwp + nfu;

    // stage Q (rows >= G zero); the K / V rows the FIRST unit does not fill are zeroed below (rows a unit does not fill
    // must be finite; later units find the rows of earlier ones there)
    for (int i = t; i < 16 * kRowStride / 8; i += 128) reinterpret_cast<uint4*>(Qs)[i] = make_uint4(0, 0, 0, 0);
    for (int i = t; i < 16 * kPStride / 8; i += 128) reinterpret_cast<uint4*>(Ps)[i] = make_uint4(0, 0, 0, 0);
    if (t < 8) { s_m[t] = -INFINITY; s_l[t] = 0.f; }
    __syncthreads();
    for (int i = t; i < G * 16; i += 128) {
        const int h = i >> 4, c = i & 15;
        *reinterpret_cast<uint4*>(Qs + h * kRowStride + c * 8) =
            *reinterpret_cast<const uint4*>(p.q + ((size_t)b * g.Hq + (size_t)kv * G + h) * kD + c * 8);
    }
    __syncthreads();
    // Both products put the long side on the M side of mma.sync and the (up to 8) query heads of the kv head on its N
    // side: S^T = K Q^T (16 keys x 8 heads per instruction) and O^T = V^T P^T (16 dims x 8 heads), 16 instructions
    // per warp and unit of 64 keys instead of the 32 of the heads-as-rows arrangement, which left 11 of 16 rows unused
    // at five heads (the kernel is bound by its mma.sync and instruction stream, not by memory).
    static_assert(G <= 8, "the heads of a kv head are the N side of the instruction");
    uint32_t qb[4][4];   // B fragments of Q^T: [pair of k-steps][b0, b1 of the first, b0, b1 of the second]
    {
        const int row = lane & 7, col = (lane >> 3) * 8;
#pragma unroll
        for (int kp = 0; kp < 4; kp++) ldsm_x4(qb[kp], smem_u32(Qs + row * kRowStride + kp * 32 + col));
    }
    float o[2][4];       // O^T[dims 32 warp + 16 mt + gq (and + 8)][heads 2 tq, 2 tq + 1]
#pragma unroll
    for (int mt = 0; mt < 2; mt++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[mt][e] = 0.f;
    if (t < 8) s_aold[t] = 0.f;

    // Row pointers of a unit (window page, far block's tokens, or 64 pooled far blocks) into rk / rv; returns its rows.
    // The page (and far block) of a unit, fetched one unit ahead of its use: two dependent loads (selected block -> page
    // table) that would otherwise sit between every two units of a CTA. (Pooled far blocks: one block per thread, fetched
    // where they are used.)
    auto fetch_idx = [&](int u, int& page_raw, int& tok0) {
        page_raw = 0;
        tok0 = 0;
        if (u >= U) return;
        if (u < nwp) {
            page_raw = p.table[b * g.max_pages + wp0 + u];
        } else if (g.far_tokens) {
            tok0 = sel[u - nwp] * g.C;
            page_raw = p.table[b * g.max_pages + tok0 / kPage];
        }
    };
    auto setup_unit = [&](int u, const __nv_bfloat16** rk, const __nv_bfloat16** rv, int page_raw, int tok0) -> int {
        int nrows;
        if (u < nwp) {
            const int page = checked_page(page_raw, p.n_pages);
            const int ra = u == 0 ? lo % kPage : 0;
            const int rb = u == nwp - 1 ? pos % kPage : kPage - 1;
            nrows = rb - ra + 1;
            if (t < nrows) {
                const size_t off = (((size_t)page * g.KVH + kv) * kPage + ra + t) * kD;
                rk[t] = p.K + off;
                rv[t] = p.V + off;
            }
        } else if (g.far_tokens) {
            const int page = checked_page(page_raw, p.n_pages);
            nrows = g.C;
            if (t < nrows) {
                const size_t off = (((size_t)page * g.KVH + kv) * kPage + tok0 % kPage + t) * kD;
                rk[t] = p.K + off;
                rv[t] = p.V + off;
            }
        } else {
            const int f0 = (u - nwp) * kPage;
            nrows = min(kPage, nf - f0);
            if (t < nrows) {
                const int j = sel[f0 + t];
                const int page = checked_page(p.table[b * g.max_pages + (j / spp)], p.n_pages);
                const size_t off = (((size_t)page * g.KVH + kv) * spp + j % spp) * kD;
                rk[t] = p.PK + off;
                rv[t] = p.PV + off;
            }
        }
        return nrows;
    };
    auto issue_rows = [&](__nv_bfloat16* tile, const __nv_bfloat16* const* rows, int nrows) {
        for (int i = t; i < nrows * 16; i += 128) {
            const int r = i >> 4, cch = i & 15;
            cp_async16(tile + r * kRowStride + cch * 8, rows[r] + cch * 8);
        }
        cp_async_commit();   // (one group per tile and unit, empty when there is nothing to fetch: the counts below rely on it)
    };

    // K and V of a unit travel as separate groups: Q K^T starts when K is in, V lands during the softmax; the next
    // unit's K is requested as soon as this unit's scores are out, its V as soon as this unit's P V is done.
    int nrows = 0, cur = 0;
    AT_T(p0);
    int pg = 0, tk = 0;
    fetch_idx(split, pg, tk);
    if (split < U) nrows = setup_unit(split, rowK[0], rowV[0], pg, tk);
    fetch_idx(split + p.nsplit, pg, tk);   // (used at the top of the first iteration)
    for (int i = nrows * (kRowStride / 8) + t; i < kPage * kRowStride / 8; i += 128) {
        reinterpret_cast<uint4*>(Ks)[i] = make_uint4(0, 0, 0, 0);
        reinterpret_cast<uint4*>(Vs)[i] = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
    AT_T(p1);
    AT_ACC(0, tr_start, p0); AT_ACC(1, p0, p1);
    issue_rows(Ks, rowK[0], nrows);
    issue_rows(Vs, rowV[0], nrows);
#if defined(VK_TRACE) && VK_TRACE == 7
    int tr_units = 0;
#endif
    for (int u = split; u < U; u += p.nsplit, cur ^= 1) {
        const int un = u + p.nsplit;
        int nrows_next = 0;
        AT_T(u0);
        if (un < U) nrows_next = setup_unit(un, rowK[cur ^ 1], rowV[cur ^ 1], pg, tk);
        fetch_idx(un + p.nsplit, pg, tk);   // (on its way during this unit's arithmetic)
        AT_T(u1);
        cp_async_wait1();   // K of this unit (V may still be on its way)
        __syncthreads();
        AT_T(u2);
        AT_ACC(2, u0, u1); AT_ACC(3, u1, u2);
        // ---- S^T = K Q^T: warp w takes keys 16 w .. 16 w + 15 (the M side), all heads (the N side)
        {
            float sa[4] = {0.f, 0.f, 0.f, 0.f};   // keys 16 w + gq (and + 8) x heads 2 tq, 2 tq + 1
            const uint32_t kaddr = smem_u32(Ks + (16 * warp + (lane & 7) + ((lane >> 3) & 1) * 8) * kRowStride + (lane >> 4) * 8);
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {
                uint32_t ka[4];
                ldsm_x4(ka, kaddr + ks * 32);
                mma16816(sa, ka, qb[ks >> 1][2 * (ks & 1)], qb[ks >> 1][2 * (ks & 1) + 1]);
            }
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int h = 2 * tq + (e & 1), key = 16 * warp + gq + 8 * (e >> 1);
                if (h < G) sc[h * kPage + key] = key < nrows ? sa[e] * p.scale : -INFINITY;
            }
        }
        __syncthreads();
        issue_rows(Ks, rowK[cur ^ 1], nrows_next);   // every warp is done with this unit's K
        // ---- softmax pieces: sixteen lanes per head (thread t: head t / 16, keys 4 (t % 16) ..): all heads in one pass
        {
            const int h = t >> 4, sub = t & 15;
            if (h < G) {   // (uniform over the sixteen lanes of a head)
                const float4 s4 = *reinterpret_cast<const float4*>(&sc[h * kPage + 4 * sub]);
                float mx = fmaxf(fmaxf(s4.x, s4.y), fmaxf(s4.z, s4.w));   // finite for the half-warp: a unit has at least one row
                const float m_old = s_m[h];
                const uint32_t half_mask = 0xFFFFu << (lane & 16);
#pragma unroll
                for (int off = 8; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(half_mask, mx, off));
                const float m_new = fmaxf(m_old, mx);
                const float p0 = bfr(__expf(s4.x - m_new)), p1 = bfr(__expf(s4.y - m_new));
                const float p2 = bfr(__expf(s4.z - m_new)), p3 = bfr(__expf(s4.w - m_new));
                uint2 pk;
                pk.x = pack_bf2(p0, p1);
                pk.y = pack_bf2(p2, p3);
                *reinterpret_cast<uint2*>(Ps + h * kPStride + 4 * sub) = pk;
                float sum = (p0 + p1) + (p2 + p3);
#pragma unroll
                for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(half_mask, sum, off);
                __syncwarp(half_mask);   // (every lane has read s_m[h])
                if (sub == 0) {
                    const float a_old = m_old == -INFINITY ? 0.f : __expf(m_old - m_new);
                    s_l[h] = s_l[h] * a_old + sum;
                    s_m[h] = m_new;
                    s_aold[h] = a_old;
                }
            }
        }
        AT_T(u3);
        cp_async_wait1();   // V of this unit (the next unit's K may still be on its way)
        __syncthreads();
        AT_T(u4);
        AT_ACC(4, u2, u3); AT_ACC(5, u3, u4);
        // ---- O^T = O^T * a_old + V^T P^T: warp w takes dims 32 w .. 32 w + 31 (the M side, two tiles of 16)
        {
            const float a0 = s_aold[2 * tq], a1 = s_aold[2 * tq + 1];
#pragma unroll
            for (int mt = 0; mt < 2; mt++) { o[mt][0] *= a0; o[mt][1] *= a1; o[mt][2] *= a0; o[mt][3] *= a1; }
            // A = V^T through transposing loads of V's [key][dim] tile; B = P^T from the probability tile's [head][key] rows
            const uint32_t vaddr = smem_u32(Vs + ((lane & 7) + (lane >> 4) * 8) * kRowStride + 32 * warp + ((lane >> 3) & 1) * 8);
            const uint32_t paddr = smem_u32(Ps + (lane & 7) * kPStride + (lane >> 3) * 8);
#pragma unroll
            for (int kp = 0; kp < 2; kp++) {   // two k-steps of 16 keys per load of P^T
                uint32_t pb[4];
                ldsm_x4(pb, paddr + kp * 64);
#pragma unroll
                for (int kk = 0; kk < 2; kk++) {
                    const int ks = 2 * kp + kk;
#pragma unroll
                    for (int mt = 0; mt < 2; mt++) {
                        uint32_t va[4];
                        ldsm_x4_t(va, vaddr + (uint32_t)(ks * 16 * kRowStride + mt * 16) * 2u);
                        mma16816(o[mt], va, pb[2 * kk], pb[2 * kk + 1]);
                    }
                }
            }
        }
        __syncthreads();   // every warp is done with this unit's V
        issue_rows(Vs, rowV[cur ^ 1], nrows_next);
        nrows = nrows_next;
#if defined(VK_TRACE) && VK_TRACE == 7
        { const long long u5 = clock64(); tr[6] += u5 - u4; tr_units++; }
#endif
    }
    cp_async_wait0();
    __syncthreads();
#if defined(VK_TRACE) && VK_TRACE == 7
    if (t == 0) {
        long long* o = g_vk_trace + (((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) & 4095) * 16;
        for (int q = 0; q < 7; q++) o[q] = tr[q];
        o[7] = clock64() - tr_start; o[8] = tr_units; o[9] = U;
    }
#endif
    float* out = p.part + (((size_t)b * g.KVH + kv) * p.nsplit + split) * G * (kD + 2);
#pragma unroll
    for (int mt = 0; mt < 2; mt++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int h = 2 * tq + (e & 1), dim = 32 * warp + 16 * mt + gq + 8 * (e >> 1);
            if (h < G) out[h * (kD + 2) + dim] = o[mt][e];
        }
    if (t < G) { out[t * (kD + 2) + kD] = s_m[t]; out[t * (kD + 2) + kD + 1] = s_l[t]; }
}

bool g_attend_tc = true;

template <int G>
cudaError_t launch_attend(const AttendParams& p, int B, cudaStream_t stream) {
    if (g_attend_tc) return vk_launch(attend_decode_tc_kernel<G>, dim3(p.nsplit, p.g.KVH, B), dim3(128), 0, stream, p);
    return vk_launch(attend_decode_kernel<G>, dim3(p.nsplit, p.g.KVH, B), dim3(128), 0, stream, p);
}

}  // namespace

extern "C" {

struct vk_attn_geom {
    int Hq, KVH, D, W, C, topk, IH, Di, NS, far_tokens, max_pages, n_pages;
};

static int geom_ok(const vk_attn_geom* gm) {
    if (gm->D != kD || gm->Hq <= 0 || gm->KVH <= 0 || gm->Hq % gm->KVH != 0 || gm->Hq / gm->KVH > 8) return 0;
    if (gm->W > 0) {
        if (gm->C <= 0 || kPage % gm->C != 0 || gm->W % gm->C != 0 || gm->topk <= 0) return 0;
        if (gm->NS != 1 && gm->NS != gm->KVH) return 0;
        if (gm->NS == 1 && (gm->Di != kD || gm->IH <= 0 || gm->IH > 8)) return 0;
    }
    return 1;
}
static AttnGeom to_geom(const vk_attn_geom* gm) {
    AttnGeom g = {gm->Hq, gm->KVH, gm->W, gm->C, gm->topk, gm->IH, gm->Di, gm->W > 0 ? gm->NS : 0, gm->far_tokens, gm->max_pages};
    return g;
}

int vk_batch_step_begin(const int* pos, int* table, int max_pages, int* free_list, int* free_top, int* desc, int B, int W,
                        int C, int topk, cudaStream_t stream) {
    if (B <= 0 || max_pages <= 0 || (W > 0 && C <= 0)) return VK_EINVAL;
    return (int)vk_launch(batch_step_begin_kernel, dim3(1), dim3(32), 0, stream, pos, table, max_pages, free_list, free_top,
                          desc, B, W, C, topk);
}

int vk_pages_open(const int* pos, const int* lens, int* table, int max_pages, const int* free_list, int* free_top, int B,
                  cudaStream_t stream) {
    if (B <= 0 || max_pages <= 0) return VK_EINVAL;
    return (int)vk_launch(pages_open_kernel, dim3(1), dim3(32), 0, stream, pos, lens, table, max_pages, free_list, free_top, B);
}

int vk_pages_release(const int* rows, const int* first, const int* last, int n, int reverse, int* table, int max_pages,
                     int* free_list, int* free_top, int n_pages, cudaStream_t stream) {
    if (n <= 0 || max_pages <= 0 || n_pages <= 0) return VK_EINVAL;
    return (int)vk_launch(pages_release_kernel, dim3(1), dim3(32), 0, stream, rows, first, last, n, reverse, table, max_pages,
                          free_list, free_top, n_pages);
}

int vk_batch_step_end(int* pos, int* parity, int B, cudaStream_t stream) {
    if (B <= 0) return VK_EINVAL;
    return (int)vk_launch(batch_step_end_kernel, dim3((B + 63) / 64), dim3(64), 0, stream, pos, parity, B);
}

int vk_attn_prep_chunk(const vk_attn_geom* gm, const void* proj, int ldp, int off_k, int off_v, const void* idxq, const void* idxk,
                       const void* q_norm, const void* k_norm, const void* idx_norm, const int* pos, const int* table, void* q,
                       void* qi, void* K, void* V, void* PK, void* PV, void* BK, void* IK, int B, int rope_dims,
                       double rope_theta, float eps, int mode, const int* row_map, void* ikc, const int* first_pos,
                       cudaStream_t stream);

int vk_attn_prep(const vk_attn_geom* gm, const void* proj, int ldp, int off_k, int off_v, const void* idxq, const void* idxk,
                 const void* q_norm, const void* k_norm, const void* idx_norm, const int* pos, const int* table, void* q,
                 void* qi, void* K, void* V, void* PK, void* PV, void* BK, void* IK, int B, int rope_dims, double rope_theta,
                 float eps, cudaStream_t stream) {
    return vk_attn_prep_chunk(gm, proj, ldp, off_k, off_v, idxq, idxk, q_norm, k_norm, idx_norm, pos, table, q, qi, K, V, PK, PV,
                              BK, IK, B, rope_dims, rope_theta, eps, 0, nullptr, nullptr, nullptr, stream);
}

// The same for rows that are several positions of one sequence (a verify window, a prefill chunk): a row's block may
// then be closed by a position whose neighbours are written by other rows of the same launch, so the caller writes all
// rows first (mode 1) and pools in a second launch (mode 2). row_map names the cache row whose open-block indexer keys
// a row shares. In indexer mode the rows' own indexer keys go to ikc [B, Di] and first_pos [B] tells where the chunk
// began for the row's sequence (see PrepParams); the caller moves the open block's keys into the ring afterwards.
int vk_attn_prep_chunk(const vk_attn_geom* gm, const void* proj, int ldp, int off_k, int off_v, const void* idxq, const void* idxk,
                       const void* q_norm, const void* k_norm, const void* idx_norm, const int* pos, const int* table, void* q,
                       void* qi, void* K, void* V, void* PK, void* PV, void* BK, void* IK, int B, int rope_dims,
                       double rope_theta, float eps, int mode, const int* row_map, void* ikc, const int* first_pos,
                       cudaStream_t stream) {
    if (mode == 0 && ikc != nullptr) return VK_EINVAL;
    if (ikc != nullptr && first_pos == nullptr) return VK_EINVAL;
    if (!geom_ok(gm) || B <= 0 || rope_dims % 8 != 0 || rope_dims > kD || mode < 0 || mode > 2) return VK_EINVAL;
    PrepParams p = {};
    p.mode = mode; p.row_map = row_map; p.ikc = (__nv_bfloat16*)ikc; p.first_pos = first_pos;
    p.proj = (const __nv_bfloat16*)proj; p.idxq = (const __nv_bfloat16*)idxq; p.idxk = (const __nv_bfloat16*)idxk;
    p.q_norm = (const __nv_bfloat16*)q_norm; p.k_norm = (const __nv_bfloat16*)k_norm; p.idx_norm = (const __nv_bfloat16*)idx_norm;
    p.pos = pos; p.table = table; p.q = (__nv_bfloat16*)q; p.qi = (__nv_bfloat16*)qi;
    p.K = (__nv_bfloat16*)K; p.V = (__nv_bfloat16*)V; p.PK = (__nv_bfloat16*)PK; p.PV = (__nv_bfloat16*)PV;
    p.BK = (__nv_bfloat16*)BK; p.IK = (__nv_bfloat16*)IK;
    p.ldp = ldp; p.off_k = off_k; p.off_v = off_v; p.n_pages = gm->n_pages; p.rope_dims = rope_dims;
    p.log2_theta = log2(rope_theta); p.eps = eps; p.g = to_geom(gm);
    const int nheads = p.g.Hq + 2 * p.g.KVH + (idxq ? p.g.IH + 1 : 0);
    return (int)vk_launch(attn_prep_kernel, dim3(B, (nheads + 7) / 8), dim3(256), 0, stream, p);
}

int vk_attn_prep_rows(const vk_attn_geom* gm, const void* proj, int ldp, int off_k, int off_v, const void* idxq, const void* idxk,
                      const void* q_norm, const void* k_norm, const void* idx_norm, const int* pos, const int* table, void* q,
                      void* qi, void* K, void* V, void* PK, void* PV, void* BK, void* IK, int B, int rope_dims,
                      double rope_theta, float eps, int mode, const int* row_map, cudaStream_t stream) {
    return vk_attn_prep_chunk(gm, proj, ldp, off_k, off_v, idxq, idxk, q_norm, k_norm, idx_norm, pos, table, q, qi, K, V, PK, PV,
                              BK, IK, B, rope_dims, rope_theta, eps, mode, row_map, nullptr, nullptr, stream);
}

// The selection kernel's shared-memory path needs more than the default 48 KB of dynamic shared memory: opt in once
// per device (the first selection call on a device must therefore come outside stream capture).
static bool select_configured() {
    static std::atomic<bool> done[64];
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (!done[dev].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(bcsa_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSelectSmem) != cudaSuccess)
            return false;
        done[dev].store(true, std::memory_order_release);
    }
    return true;
}

int vk_attn_configure(void) { return select_configured() ? VK_OK : VK_EINVAL; }

size_t vk_bcsa_select_scratch_bytes(const vk_attn_geom* gm, int B, int max_blocks) {
    return (size_t)B * (gm->NS > 0 ? gm->NS : 1) * max_blocks * 4;
}

int vk_bcsa_select(const vk_attn_geom* gm, const void* q, const void* keys, const int* pos, const int* table, void* scratch,
                   int max_blocks, int* sel, int* nsel, int B, cudaStream_t stream) {
    if (!geom_ok(gm) || gm->W <= 0 || B <= 0 || max_blocks <= 0) return VK_EINVAL;
    SelectParams p = {};
    p.q = (const __nv_bfloat16*)q; p.keys = (const __nv_bfloat16*)keys; p.pos = pos; p.table = table;
    p.scratch = (uint32_t*)scratch; p.sel = sel; p.nsel = nsel; p.cap = max_blocks; p.n_pages = gm->n_pages;
    p.scale = (float)(1.0 / sqrt((double)kD)); p.g = to_geom(gm);
    if (!select_configured()) return VK_EINVAL;
    return (int)vk_launch(bcsa_select_kernel, dim3(p.g.NS, B), dim3(256), kSelectSmem, stream, p);
}

// ---- far-block selection for callers that cannot allocate
// Fixed capacity of the built-in scratch: 16 rows x 8 selection groups x 2048 blocks per row (1 MiB, held by every
// GPU that loads the library until the process exits).
namespace {
constexpr int kStaticRows = 16, kStaticGroups = 8, kStaticBlocks = 2048;
static __device__ __align__(256) uint32_t g_select_scratch[kStaticRows * kStaticGroups * kStaticBlocks];
std::atomic<uint32_t*> g_select_scratch_addr[64];  // device address of the array, per device ordinal (host-side cache)
}  // namespace

int vk_bcsa_select_static(const vk_attn_geom* gm, const void* q, const void* keys, const int* pos, const int* table, int* sel,
                          int* nsel, int B, cudaStream_t stream) {
    if (!geom_ok(gm) || gm->W <= 0 || B <= 0) return VK_EINVAL;
    const long long blocks = (long long)gm->max_pages * (kPage / gm->C);
    if (gm->max_pages <= 0) return VK_EINVAL;
    if (B > kStaticRows || gm->NS > kStaticGroups || blocks > kStaticBlocks) return VK_ETOOBIG;
    int dev = -1;
    VK_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return VK_EINVAL;
    uint32_t* scratch = g_select_scratch_addr[dev].load(std::memory_order_acquire);
    if (scratch == nullptr) {
        // In host code the array's name is only a handle; the kernel needs the address the current device gave it.
        // (Two host threads that both find the slot empty look the same address up twice: harmless.)
        void* addr = nullptr;
        VK_CUDA(cudaGetSymbolAddress(&addr, g_select_scratch));
        scratch = (uint32_t*)addr;
        g_select_scratch_addr[dev].store(scratch, std::memory_order_release);
    }
    SelectParams p = {};
    p.q = (const __nv_bfloat16*)q; p.keys = (const __nv_bfloat16*)keys; p.pos = pos; p.table = table;
    // (cap = this geometry's block count, as vk_bcsa_select gets it: a position beyond the row's page table is then
    // reported instead of indexing past the table; rows are (b * NS + ns) * cap apart, inside the array for every
    // shape that passed the check above)
    p.scratch = scratch; p.sel = sel; p.nsel = nsel; p.cap = (int)blocks; p.n_pages = gm->n_pages;
    p.scale = (float)(1.0 / sqrt((double)kD)); p.g = to_geom(gm);
    if (!select_configured()) return VK_EINVAL;
    return (int)vk_launch(bcsa_select_kernel, dim3(p.g.NS, B), dim3(256), kSelectSmem, stream, p);
}

// 1 (default): both attention products on the tensor cores; 0: the scalar kernel (kept as a cross-check)
void vk_attend_set_tensor_cores(int on) { g_attend_tc = on != 0; }

size_t vk_attend_scratch_bytes(const vk_attn_geom* gm, int B, int nsplit) {
    return (size_t)B * gm->Hq * nsplit * (kD + 2) * 4;
}

int vk_attend_decode(const vk_attn_geom* gm, const void* q, const void* K, const void* V, const void* PK, const void* PV,
                     const int* pos, const int* table, const int* sel, const int* nsel, const void* proj, int ldp,
                     void* part, int nsplit, void* out, void* xrec_out, int B, cudaStream_t stream) {
    if (!geom_ok(gm) || B <= 0 || nsplit <= 0 || (xrec_out != nullptr && B > 16)) return VK_EINVAL;
    AttendParams p = {};
    p.q = (const __nv_bfloat16*)q; p.K = (const __nv_bfloat16*)K; p.V = (const __nv_bfloat16*)V;
    p.PK = (const __nv_bfloat16*)PK; p.PV = (const __nv_bfloat16*)PV; p.pos = pos; p.table = table;
    p.sel = gm->W > 0 ? sel : nullptr; p.nsel = nsel; p.part = (float*)part; p.nsplit = nsplit; p.n_pages = gm->n_pages;
    p.scale = (float)(1.0 / sqrt((double)kD)); p.g = to_geom(gm);
    cudaError_t e;
    switch (gm->Hq / gm->KVH) {
        case 1: e = launch_attend<1>(p, B, stream); break;
        case 2: e = launch_attend<2>(p, B, stream); break;
        case 3: e = launch_attend<3>(p, B, stream); break;
        case 4: e = launch_attend<4>(p, B, stream); break;
        case 5: e = launch_attend<5>(p, B, stream); break;
        case 6: e = launch_attend<6>(p, B, stream); break;
        case 8: e = launch_attend<8>(p, B, stream); break;
        default: return VK_EINVAL;
    }
    if (e != cudaSuccess) return (int)e;
    return (int)vk_launch(attend_merge_kernel, dim3(gm->Hq, B), dim3(128), 0, stream, (const float*)part,
                          (const __nv_bfloat16*)proj, ldp, (__nv_bfloat16*)out, (uint8_t*)xrec_out, gm->Hq, gm->KVH, nsplit);
}

}  // extern "C"
