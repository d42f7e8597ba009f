// Attention for rows that are consecutive positions of one sequence (a verify window of T drafted tokens, a prefill
// chunk): tiles of up to 16 query positions x the G query heads of a kv head share one pass over the keys. Replaces
// bcsa_verify.attend (bcsa_verify.py:278-317: G * T query rows per kv head, the ring read once, the keys split over
// several thread groups and merged), far_union + bcsa_attend (kernels.py:931-1020, :1023-1165: a block of queries
// attends the UNION of its queries' selected far blocks, every query masked to its own) and the dense layer of
// batch_spec._dense (batch_spec.py:50-64) on the paged cache.
//
// One CTA per (split, kv head, tile). Warp h of the CTA owns query head h of the kv head: its 16 x 128 Q tile (row =
// query position of the tile) stays in registers as mma A fragments, S = Q K^T for a unit of up to 64 keys is formed in
// registers, the probabilities go straight from the accumulator layout into the A operand of P V (no shared-memory
// round trip), O (16 x 128 fp32) and the running max / sum stay in registers: the flash-attention-2 arrangement. The
// units' K and V rows are staged in shared memory once per CTA and read by all G warps; next unit's K is requested
// while this unit's softmax runs, its V while P V runs (cp.async groups, as in attend_decode_tc_kernel).
//
// Keys of a tile whose first query stands at position p0 and whose last at p1:
//   window   positions max(0, p0 - W + 1) .. p1 (dense layers: 0 .. p1), page by page; query at position p sees
//            max(0, p - W + 1) .. p of them (sliding window + causal order inside the chunk);
//   far      the union of the tile's queries' selected blocks (ascending), each block visible to the queries that
//            selected it: a bit mask per block, built in shared memory from the queries' sorted lists. Far keys are
//            the blocks' tokens (64-token-block form) or their pooled rows (reference form), as in the decode kernel.
// Output: the same per-(row, kv head, split) partial layout as the decode kernel's, so attend_merge_kernel finishes the
// rows (merge of the splits, division, sigmoid gate).
#include "common.cuh"

namespace {

constexpr int kTQ = 16;   // query positions per tile

struct ChunkAttendParams {
    const __nv_bfloat16* q;     // [R, Hq, D]
    const __nv_bfloat16 *K, *V, *PK, *PV;
    const int* pos;             // [R] position of every virtual row
    const int* table;           // [R, max_pages] (all rows of a request carry the same table)
    const int* sel;             // [R, NS, topk] or null
    const int* nsel;            // [R, NS]
    const int* tile_first;      // [tiles] first virtual row
    const int* tile_count;      // [tiles] rows (1..16)
    float* part;                // [R, KVH, nsplit, G, D + 2]
    int nsplit, n_pages, nv_cap, u_cap;
    float scale;
    AttnGeom g;
};

__device__ __forceinline__ uint32_t pack2(float a, float b) { return pack_bf2(a, b); }

template <int G>
__global__ void __launch_bounds__(32 * G) attend_chunk_kernel(const ChunkAttendParams p) {
    extern __shared__ __align__(16) uint8_t dsm[];
    __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(dsm);
    __nv_bfloat16* Vs = Ks + kPage * kRowStride;
    uint32_t* memb = reinterpret_cast<uint32_t*>(Vs + kPage * kRowStride);   // [nv_cap / 2 + 1]: 16-bit query masks per block
    uint32_t* ulist = memb + (p.nv_cap / 2 + 1);                              // [u_cap] union of selected blocks, ascending
    __shared__ const __nv_bfloat16* rowK[2][kPage];
    __shared__ const __nv_bfloat16* rowV[2][kPage];
    __shared__ __align__(16) int kinfo[2][kPage];   // >= 0: the key's position (window); < 0: far key, low 16 bits = queries that see it
    __shared__ int s_count, s_base;
    __shared__ int wcount[8];
    pdl_launch_dependents();
    pdl_wait();
    const AttnGeom& g = p.g;
    const int split = blockIdx.x, kv = blockIdx.y, tile = blockIdx.z;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31, nthr = 32 * G;
    const int gq = lane >> 2, tq = lane & 3;
    const int v0 = p.tile_first[tile], n = p.tile_count[tile];
    const int p0 = p.pos[v0], p1 = p0 + n - 1;
    const int lo_min = g.W > 0 ? max(0, p0 - g.W + 1) : 0;
    const int wp0 = lo_min / kPage, nwp = p1 / kPage - wp0 + 1;
    const int ns = g.NS > 1 ? kv : 0;
    const int spp = g.W > 0 ? kPage / g.C : 1;
    const int* tab = p.table + (size_t)v0 * g.max_pages;

    // zero the tiles once (rows a unit does not fill must stay finite)
    for (int i = t; i < 2 * kPage * kRowStride / 8; i += nthr) reinterpret_cast<uint4*>(Ks)[i] = make_uint4(0, 0, 0, 0);

    // ---- the union of the queries' far blocks and who sees which
    int nu = 0;
    if (g.W > 0 && p.sel != nullptr && g.NS > 0) {
        const int nv_max = max(0, (p1 - g.W + 1) / g.C);
        if (nv_max > p.nv_cap) {
            if (t == 0) vk_set_status(VK_ST_BAD_INDEX);
            return;
        }
        for (int i = t; i < nv_max / 2 + 1; i += nthr) memb[i] = 0u;
        if (t == 0) { s_count = 0; s_base = 0; }
        __syncthreads();
        for (int i = t; i < n * g.topk; i += nthr) {
            const int qi = i / g.topk, e = i % g.topk;
            const int row = v0 + qi;
            if (e < p.nsel[row * g.NS + ns]) {
                const int j = p.sel[((size_t)row * g.NS + ns) * g.topk + e];
                if (j >= 0 && j < nv_max) atomicOr(&memb[j >> 1], (1u << qi) << (16 * (j & 1)));
                else vk_set_status(VK_ST_BAD_INDEX);
            }
        }
        __syncthreads();
        // ordered compaction: blocks with a non-empty mask, ascending
        for (int j0 = 0; j0 < nv_max; j0 += nthr) {
            const int j = j0 + t;
            const bool take = j < nv_max && ((memb[j >> 1] >> (16 * (j & 1))) & 0xFFFFu) != 0u;
            const uint32_t bal = __ballot_sync(0xffffffffu, take);
            if (lane == 0) wcount[warp] = __popc(bal);
            __syncthreads();
            int off = s_base;
            for (int w = 0; w < warp; w++) off += wcount[w];
            if (take) {
                const int r = off + __popc(bal & ((1u << lane) - 1u));
                if (r < p.u_cap) ulist[r] = (uint32_t)j;
            }
            __syncthreads();
            if (t == 0) {
                int tot = 0;
                for (int w = 0; w < G; w++) tot += wcount[w];
                s_base += tot;
            }
            __syncthreads();
        }
        nu = min(s_base, p.u_cap);
    }
    const int nfu = g.far_tokens ? nu : (nu + kPage - 1) / kPage;
    const int U = nwp + nfu;

    // ---- this warp's Q tile as A fragments: row = query of the tile (rows >= n are zero), 8 k-steps over the head dim
    uint32_t qf[8][4];
    {
        const int head = kv * G + warp;
        const __nv_bfloat16* q0 = p.q + ((size_t)(v0 + gq) * g.Hq + head) * kD;
        const __nv_bfloat16* q1 = p.q + ((size_t)(v0 + gq + 8) * g.Hq + head) * kD;
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
            const int c = ks * 16 + 2 * tq;
            qf[ks][0] = gq < n ? *reinterpret_cast<const uint32_t*>(q0 + c) : 0u;
            qf[ks][1] = gq + 8 < n ? *reinterpret_cast<const uint32_t*>(q1 + c) : 0u;
            qf[ks][2] = gq < n ? *reinterpret_cast<const uint32_t*>(q0 + c + 8) : 0u;
            qf[ks][3] = gq + 8 < n ? *reinterpret_cast<const uint32_t*>(q1 + c + 8) : 0u;
        }
    }
    // per-row facts of the two rows this thread holds (queries gq and gq + 8)
    const int qa = gq, qb = gq + 8;
    const int pa_pos = p0 + qa, pb_pos = p0 + qb;
    const int lo_a = g.W > 0 ? max(0, pa_pos - g.W + 1) : 0, lo_b = g.W > 0 ? max(0, pb_pos - g.W + 1) : 0;
    const bool va = qa < n, vb = qb < n;

    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; i++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[i][e] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

    // rows of unit u -> row pointers and key facts in buffer `buf`; returns the unit's row count
    auto setup_unit = [&](int u, int buf) -> int {
        int nrows;
        if (u < nwp) {
            const int page = checked_page(tab[wp0 + u], p.n_pages);
            const int ra = u == 0 ? lo_min % kPage : 0;
            const int rb = u == nwp - 1 ? p1 % kPage : kPage - 1;
            nrows = rb - ra + 1;
            for (int i = t; i < kPage; i += nthr) {
                if (i < nrows) {
                    const size_t off = (((size_t)page * g.KVH + kv) * kPage + ra + i) * kD;
                    rowK[buf][i] = p.K + off;
                    rowV[buf][i] = p.V + off;
                    kinfo[buf][i] = (wp0 + u) * kPage + ra + i;
                } else {
                    kinfo[buf][i] = (int)0x80000000;
                }
            }
        } else if (g.far_tokens) {
            const int j = (int)ulist[u - nwp];
            const int tok0 = j * g.C;
            const int page = checked_page(tab[tok0 / kPage], p.n_pages);
            const int mask = (int)((memb[j >> 1] >> (16 * (j & 1))) & 0xFFFFu);
            nrows = g.C;
            for (int i = t; i < kPage; i += nthr) {
                if (i < nrows) {
                    const size_t off = (((size_t)page * g.KVH + kv) * kPage + tok0 % kPage + i) * kD;
                    rowK[buf][i] = p.K + off;
                    rowV[buf][i] = p.V + off;
                    kinfo[buf][i] = (int)(0x80000000u | (uint32_t)mask);
                } else {
                    kinfo[buf][i] = (int)0x80000000;
                }
            }
        } else {
            const int f0 = (u - nwp) * kPage;
            nrows = min(kPage, nu - f0);
            for (int i = t; i < kPage; i += nthr) {
                if (i < nrows) {
                    const int j = (int)ulist[f0 + i];
                    const int page = checked_page(tab[j / spp], p.n_pages);
                    const size_t off = (((size_t)page * g.KVH + kv) * spp + j % spp) * kD;
                    rowK[buf][i] = p.PK + off;
                    rowV[buf][i] = p.PV + off;
                    kinfo[buf][i] = (int)(0x80000000u | ((memb[j >> 1] >> (16 * (j & 1))) & 0xFFFFu));
                } else {
                    kinfo[buf][i] = (int)0x80000000;
                }
            }
        }
        return nrows;
    };
    auto issue_rows = [&](__nv_bfloat16* tilep, const __nv_bfloat16* const* rows, int nrows) {
        for (int i = t; i < nrows * 16; i += nthr) {
            const int r = i >> 4, cch = i & 15;
            cp_async16(tilep + r * kRowStride + cch * 8, rows[r] + cch * 8);
        }
        cp_async_commit();   // (one group per tile and unit, empty when there is nothing to fetch: the counts below rely on it)
    };

    int nrows = 0, cur = 0;
    if (split < U) nrows = setup_unit(split, 0);
    __syncthreads();
    issue_rows(Ks, rowK[0], nrows);
    issue_rows(Vs, rowV[0], nrows);
    const int mat = lane >> 3, r8 = lane & 7;
    for (int u = split; u < U; u += p.nsplit, cur ^= 1) {
        const int un = u + p.nsplit;
        int nrows_next = 0;
        if (un < U) nrows_next = setup_unit(un, cur ^ 1);
        cp_async_wait1();   // K of this unit (V may still be on its way)
        __syncthreads();
        // ---- S = Q K^T: 16 queries x 64 keys per warp
        float sa[8][4];
#pragma unroll
        for (int i = 0; i < 8; i++)
#pragma unroll
            for (int e = 0; e < 4; e++) sa[i][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
#pragma unroll
            for (int np = 0; np < 4; np++) {
                uint32_t kb[4];
                ldsm_x4(kb, smem_u32(Ks + (16 * np + (mat >> 1) * 8 + r8) * kRowStride + ks * 16 + (mat & 1) * 8));
                mma16816(sa[2 * np], qf[ks], kb[0], kb[1]);
                mma16816(sa[2 * np + 1], qf[ks], kb[2], kb[3]);
            }
        }
        // ---- masks and the running softmax of the two rows this thread shares with its quad
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            const int2 inf = *reinterpret_cast<const int2*>(&kinfo[cur][8 * nt + 2 * tq]);
            const int info[2] = {inf.x, inf.y};
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int ki = info[e];
                const bool far = ki < 0;
                const bool sa_vis = va && (far ? ((ki >> qa) & 1) != 0 : (ki <= pa_pos && ki >= lo_a));
                const bool sb_vis = vb && (far ? ((ki >> qb) & 1) != 0 : (ki <= pb_pos && ki >= lo_b));
                sa[nt][e] = sa_vis ? sa[nt][e] * p.scale : -INFINITY;
                sa[nt][2 + e] = sb_vis ? sa[nt][2 + e] * p.scale : -INFINITY;
                mx_a = fmaxf(mx_a, sa[nt][e]);
                mx_b = fmaxf(mx_b, sa[nt][2 + e]);
            }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        const float ms_a = mn_a == -INFINITY ? 0.f : mn_a, ms_b = mn_b == -INFINITY ? 0.f : mn_b;   // (nothing seen yet)
        const float al_a = __expf(m_a - ms_a), al_b = __expf(m_b - ms_b);                           // exp(-inf) = 0
        m_a = mn_a;
        m_b = mn_b;
        float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
#pragma unroll
            for (int e = 0; e < 2; e++) {
                sa[nt][e] = bfr(__expf(sa[nt][e] - ms_a));
                sa[nt][2 + e] = bfr(__expf(sa[nt][2 + e] - ms_b));
                sum_a += sa[nt][e];
                sum_b += sa[nt][2 + e];
            }
        }
        l_a = l_a * al_a + sum_a;   // (this thread's share of the row sums; the quad adds up at the end)
        l_b = l_b * al_b + sum_b;
        __syncthreads();            // every warp is done with this unit's K
        issue_rows(Ks, rowK[cur ^ 1], nrows_next);
#pragma unroll
        for (int i = 0; i < 16; i++) { o[i][0] *= al_a; o[i][1] *= al_a; o[i][2] *= al_b; o[i][3] *= al_b; }
        cp_async_wait1();   // V of this unit (the next unit's K may still be on its way)
        __syncthreads();
        // ---- O += P V: the probabilities as A fragments straight from the accumulator layout
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            uint32_t pa[4];
            pa[0] = pack2(sa[2 * ks][0], sa[2 * ks][1]);
            pa[1] = pack2(sa[2 * ks][2], sa[2 * ks][3]);
            pa[2] = pack2(sa[2 * ks + 1][0], sa[2 * ks + 1][1]);
            pa[3] = pack2(sa[2 * ks + 1][2], sa[2 * ks + 1][3]);
#pragma unroll
            for (int dp = 0; dp < 8; dp++) {
                uint32_t vbf[4];
                ldsm_x4_t(vbf, smem_u32(Vs + (ks * 16 + (mat & 1) * 8 + r8) * kRowStride + dp * 16 + (mat >> 1) * 8));
                mma16816(o[2 * dp], pa, vbf[0], vbf[1]);
                mma16816(o[2 * dp + 1], pa, vbf[2], vbf[3]);
            }
        }
        __syncthreads();   // every warp is done with this unit's V
        issue_rows(Vs, rowV[cur ^ 1], nrows_next);
        nrows = nrows_next;
    }
    cp_async_wait0();
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    // ---- partial results per (virtual row, kv head, split): [G][D + 2]
    if (va) {
        float* out = p.part + ((((size_t)(v0 + qa) * g.KVH + kv) * p.nsplit + split) * G + warp) * (kD + 2);
#pragma unroll
        for (int i = 0; i < 16; i++) *reinterpret_cast<float2*>(out + 8 * i + 2 * tq) = make_float2(o[i][0], o[i][1]);
        if (tq == 0) { out[kD] = m_a; out[kD + 1] = l_a; }
    }
    if (vb) {
        float* out = p.part + ((((size_t)(v0 + qb) * g.KVH + kv) * p.nsplit + split) * G + warp) * (kD + 2);
#pragma unroll
        for (int i = 0; i < 16; i++) *reinterpret_cast<float2*>(out + 8 * i + 2 * tq) = make_float2(o[i][2], o[i][3]);
        if (tq == 0) { out[kD] = m_b; out[kD + 1] = l_b; }
    }
}

template <int G>
cudaError_t launch_attend_chunk(const ChunkAttendParams& p, int n_tiles, size_t smem, cudaStream_t stream) {
    static std::atomic<size_t> configured[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (configured[dev].load(std::memory_order_acquire) < smem) {   // (opt in to more dynamic shared memory as shapes ask for it)
        e = cudaFuncSetAttribute(attend_chunk_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured[dev].store(smem, std::memory_order_release);
    }
    return vk_launch(attend_chunk_kernel<G>, dim3(p.nsplit, p.g.KVH, n_tiles), dim3(32 * G), smem, stream, p);
}

}  // namespace

extern "C" {

// Shared memory the tile kernel needs for rows whose last query sees nv_cap valid far blocks.
size_t vk_attend_chunk_smem_bytes(const vk_attn_geom* gm, int nv_cap) {
    const size_t u_cap = (size_t)(nv_cap < kTQ * gm->topk ? nv_cap : kTQ * gm->topk);
    return (size_t)2 * kPage * kRowStride * 2 + ((size_t)nv_cap / 2 + 1) * 4 + (u_cap + 1) * 4;
}

int vk_attend_chunk(const vk_attn_geom* gm, const void* q, const void* K, const void* V, const void* PK, const void* PV,
                    const int* pos, const int* table, const int* sel, const int* nsel, const int* tile_first,
                    const int* tile_count, int n_tiles, int nv_cap, const void* proj, int ldp, void* part, int nsplit, void* out,
                    int R, cudaStream_t stream) {
    if (!geom_ok(gm) || R <= 0 || n_tiles <= 0 || nsplit <= 0 || nv_cap < 0) return VK_EINVAL;
    const size_t smem = vk_attend_chunk_smem_bytes(gm, nv_cap);
    if (smem > 200 * 1024) return VK_ETOOBIG;
    ChunkAttendParams p = {};
    p.q = (const __nv_bfloat16*)q; p.K = (const __nv_bfloat16*)K; p.V = (const __nv_bfloat16*)V;
    p.PK = (const __nv_bfloat16*)PK; p.PV = (const __nv_bfloat16*)PV; p.pos = pos; p.table = table;
    p.sel = gm->W > 0 ? sel : nullptr; p.nsel = nsel; p.tile_first = tile_first; p.tile_count = tile_count;
    p.part = (float*)part; p.nsplit = nsplit; p.n_pages = gm->n_pages; p.nv_cap = nv_cap;
    p.u_cap = nv_cap < kTQ * gm->topk ? nv_cap : kTQ * gm->topk;
    p.scale = (float)(1.0 / sqrt((double)kD)); p.g = to_geom(gm);
    cudaError_t e;
    switch (gm->Hq / gm->KVH) {
        case 1: e = launch_attend_chunk<1>(p, n_tiles, smem, stream); break;
        case 2: e = launch_attend_chunk<2>(p, n_tiles, smem, stream); break;
        case 3: e = launch_attend_chunk<3>(p, n_tiles, smem, stream); break;
        case 4: e = launch_attend_chunk<4>(p, n_tiles, smem, stream); break;
        case 5: e = launch_attend_chunk<5>(p, n_tiles, smem, stream); break;
        case 6: e = launch_attend_chunk<6>(p, n_tiles, smem, stream); break;
        case 8: e = launch_attend_chunk<8>(p, n_tiles, smem, stream); break;
        default: return VK_EINVAL;
    }
    if (e != cudaSuccess) return (int)e;
    return (int)vk_launch(attend_merge_kernel, dim3(gm->Hq, R), dim3(128), 0, stream, (const float*)part,
                          (const __nv_bfloat16*)proj, ldp, (__nv_bfloat16*)out, (uint8_t*)nullptr, gm->Hq, gm->KVH, nsplit);
}

}  // extern "C"
