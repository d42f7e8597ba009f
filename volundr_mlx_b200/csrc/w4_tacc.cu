// The INT4 small-M GEMM (1..16 activation rows) as "dequantise into shared memory, accumulate in tensor memory":
//   y[m, n] = sum_k x[m, k] * bf16(s[n, k / 64] * u[n, k] + b[n, k / 64]),   fp32 accumulation,
// i.e. the activations times the dequantised weights exactly as mx.dequantize returns them (bit for bit, see the
// expansion below), the arithmetic of "dequantise, then matmul" (volundr.py:185-190 with the weights materialised).
//
// Why a second form beside w4_gemm_kernel<MT, 0>: mma.sync runs at a quarter of the tcgen05 rate on this architecture
// (one m16n8k16 per 8 cycles and scheduler) and that kernel's instruction stream holds it at 2.9 TB/s of weights. Here the tensor
// cores are driven by ONE thread (tcgen05.mma), with the roles swapped against the usual small-M arrangement: the 256
// weight rows of a superblock are the N side of the instruction, the activation rows the M side (M = 128, of which
// rows 0..15 are real: the rest of the operand is whatever follows the x record in shared memory and only reaches
// accumulator rows nobody reads), so one 9216-byte step is FOUR instructions of M 128 x N 256 x K 16 rather than the
// eight M 128 x N 16 instructions of the weights-as-M arrangement, which cost about 110 cycles each to issue whatever
// their N. The accumulator (128 lanes x 256 columns of tensor memory, fp32) stays in tensor memory across all the K
// steps of a superblock: nothing is read back per step, because the per-group scale and bias are applied BEFORE the
// product, while the codes are expanded.
//
// One CTA per SM, 20 warps:
//   warp 1        lane 0: TMA producer of the weight steps (a ring of kTaStages x 9216 bytes; the first ring-full is
//                 requested before the dependency wait: weights depend on no earlier kernel);
//                 lane 1: TMA producer of the x records, one per step, into the step's slot
//   warp 2        lane 0: per step waits for the slot's x record and its 16 expansion arrivals and issues the four
//                 tcgen05.mma; commits to the slot's "free" barrier; after the last step of a superblock segment
//                 commits to the accumulator's "ready" barrier. Two accumulators (2 x 256 columns) alternate between
//                 segments, so the next superblock starts while the last one drains.
//   warps 3, 5..19  sixteen expansion warps: 16 weight rows x 64 columns of the step each: codes -> bf16 128 + u (lop3,
//                 as in w4_gemm.cu) -> u (exact subtraction) -> fma.rn.bf16x2(u, s, b) = bf16(s u + b) with ONE rounding,
//                 stored as the B operand, K-major without swizzle: [column / 8][row 256][8]. They read only weights and
//                 therefore start before the dependency wait.
//   warps 0, 4    drain: the two warps that may read tensor-memory lanes 0..31 (a warp reads the lane quarter given by
//                 its index mod 4). Thread m < M holds activation row m; each warp takes 128 of the 256 columns in
//                 pieces of 32, and writes y (a whole superblock) or the fp32 partial sums of w4_gemm_kernel's split-K
//                 scheme (same workspace layout, same fixed order of the final addition).
// Every wait is bounded; a wait that runs out sets the status word, the CTA winds down and frees its tensor memory.
#include <cuda_bf16.h>

#include <atomic>

#include "common.cuh"

namespace {

constexpr int kTaExpWarps = 16;
constexpr int kTaWBytes = kBlocksPerSB * kChunkBytes;        // 9216
constexpr int kTaBBytes = kSBRows * 64 * 2;                  // 32 KB: [8][256][8] bf16
// MR = activation rows the A operand really holds:
//   16   the x records of the decode step (2176 bytes per 64-column group, rows 16..127 of the M = 128 operand are
//        whatever follows the record in its slot); 20 warps, drain by warps 0 and 4 (lanes 0..15 of quarter 0)
//   128  the 16 KB activation tiles of vk_w4_gemm_tile ([8][128][8] bf16 per group, rows beyond M zero): verify windows
//        and chunks of up to 128 rows; 22 warps, drain by warps 4..7 (one lane quarter each)
template <int MR> struct TaCfg {
    static constexpr int kThreads = MR == 16 ? 640 : 704;
    static constexpr int kDrainWarps = MR == 16 ? 2 : 4;
    static constexpr int kXLoad = MR == 16 ? kXRecBytes : MR * 64 * 2;      // bytes of A per step
    static constexpr int kXBytes = MR == 16 ? 2304 : MR * 64 * 2;           // ... up to the next multiple of 128
    static constexpr int kLbo = MR * 16;                                     // bytes between the operand's 16-byte units along K
    static constexpr int kSlotBytes = kXBytes + kTaBBytes;                   // a slot = the step's A operand, then its B operand
    static constexpr int kSlots = MR == 16 ? 4 : 3;
    static constexpr int kStages = MR == 16 ? 6 : 5;
    static constexpr int kPS = MR == 16 ? 16 : MR;                           // floats per row of a partial-sum slab
    static constexpr size_t kSlotOff = (size_t)kStages * kTaWBytes;
    static constexpr size_t kBarOff = kSlotOff + (size_t)kSlots * kSlotBytes;
    static constexpr int kBars = 2 * kStages + 3 * kSlots + 4;
    static constexpr size_t kSmem = kBarOff + kBars * 8;
    static_assert(kSmem <= 227 * 1024, "does not fit a CTA's shared memory");
    static_assert(7 * kLbo + 16 * 128 <= kSlotBytes, "the M = 128 operand must stay inside its slot");
};

#if defined(VK_TRACE) && VK_TRACE == 6
#define TA_T(var) const long long var = clock64()
#define TA_ACC(slot, a, b) tr[slot] += (b) - (a)
#else
#define TA_T(var) do { } while (0)
#define TA_ACC(slot, a, b) do { } while (0)
#endif

template <int N> __device__ __forceinline__ void ta_drain_sync() { asm volatile("bar.sync 2, %0;" ::"n"(N) : "memory"); }

template <int MR>
__global__ void __launch_bounds__(TaCfg<MR>::kThreads, 1) w4_tacc_kernel(const W4Params p) {
    extern __shared__ __align__(128) uint8_t smem[];
    using Cfg = TaCfg<MR>;
    constexpr int kTaSlots = Cfg::kSlots, kTaStages = Cfg::kStages, kTaSlotBytes = Cfg::kSlotBytes, kTaXBytes = Cfg::kXBytes;
    constexpr int kDrainThreads = 32 * Cfg::kDrainWarps, kPS = Cfg::kPS;
    uint8_t* slots = smem + Cfg::kSlotOff;
    uint64_t* wfull = reinterpret_cast<uint64_t*>(smem + Cfg::kBarOff);
    uint64_t* wempty = wfull + kTaStages;     // every expansion warp has the stage's codes in registers
    uint64_t* xfull = wempty + kTaStages;     // [slot] the step's x record has landed
    uint64_t* bready = xfull + kTaSlots;      // [slot] the step's dequantised weights are in place
    uint64_t* sfree = bready + kTaSlots;      // [slot] the step's MMAs have read the slot
    uint64_t* dready = sfree + kTaSlots;      // [accumulator] the segment's MMAs have finished
    uint64_t* dfree = dready + 2;             // [accumulator] both drain warps have read it
    __shared__ uint32_t s_tmem;
    __shared__ int s_last;
    __shared__ int s_fail;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    long long t0, t1;
    if (p.S > 0) {   // one K slice of one superblock
        const int asb = blockIdx.x / p.S, sl = blockIdx.x % p.S;
        t0 = (long long)asb * p.G + (long long)sl * p.G / p.S;
        t1 = (long long)asb * p.G + (long long)(sl + 1) * p.G / p.S;
    } else {
        t0 = (long long)blockIdx.x * p.T / p.P;
        t1 = (long long)(blockIdx.x + 1) * p.T / p.P;
    }
    const int n = (int)(t1 - t0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTaStages; s++) {
            mbar_init(&wfull[s], 1);
            mbar_init(&wempty[s], kTaExpWarps / 2);
        }
        for (int s = 0; s < kTaSlots; s++) {
            mbar_init(&xfull[s], 1);   // (unused: the x record's bytes are counted on bready)
            mbar_init(&bready[s], kTaExpWarps / 2 + 1);
            mbar_init(&sfree[s], 1);
        }
        for (int s = 0; s < 2; s++) {
            mbar_init(&dready[s], 1);
            mbar_init(&dfree[s], Cfg::kDrainWarps);
        }
        mbar_fence_init();
        s_fail = 0;
    }
    if (warp == 2) {   // all 512 columns: two accumulators of 256
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    if (warp == 1) {
        // ---------------------------------------------------------------- producers: lane 0 weights, lane 1 x records
        if (lane == 0) {
            const uint8_t* wsrc = p.wp + (size_t)t0 * kTaWBytes;
            const int pre = n < kTaStages ? n : kTaStages;
            for (int i = 0; i < pre; i++) {   // weights depend on no earlier kernel
                mbar_expect_tx(&wfull[i], kTaWBytes);
                tma_bulk_g2s(smem + (size_t)i * kTaWBytes, wsrc + (size_t)i * kTaWBytes, kTaWBytes, &wfull[i]);
            }
            pdl_wait();
            pdl_launch_dependents();
            int ws = 0;
            uint32_t wpar = 0;
            const uint8_t* wnext = wsrc + (size_t)pre * kTaWBytes;
            for (int i = pre; i < n; i++) {
                if (!mbar_wait(&wempty[ws], wpar)) { s_fail = 1; break; }
                fence_proxy_async_smem();   // (the expansion warps read the codes with ld.shared)
                mbar_expect_tx(&wfull[ws], kTaWBytes);
                tma_bulk_g2s(smem + (size_t)ws * kTaWBytes, wnext, kTaWBytes, &wfull[ws]);
                wnext += kTaWBytes;
                if (++ws == kTaStages) { ws = 0; wpar ^= 1u; }
            }
        } else if (lane == 1) {
            pdl_wait();   // the x records are the output of the kernel in front
            int kg = (int)(t0 % p.G);
            for (int i = 0; i < n; i++) {
                const int s = i % kTaSlots;
                if (i >= kTaSlots && !mbar_wait(&sfree[s], (uint32_t)((i / kTaSlots - 1) & 1))) { s_fail = 1; break; }
                mbar_expect_tx(&bready[s], Cfg::kXLoad);   // (one of the barrier's arrivals, plus the copy's bytes)
                tma_bulk_g2s(slots + (size_t)s * kTaSlotBytes, p.xrec + (size_t)kg * Cfg::kXLoad, Cfg::kXLoad, &bready[s]);
                kg = kg + 1 == p.G ? 0 : kg + 1;
            }
        }
    } else if (warp == 2) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0) {
            pdl_wait();   // (nothing to do before the first x record, which the kernel in front writes)
            // instruction descriptor: D fp32, A and B bf16, both K-major, N = 256 (weight rows), M = 128 (activation rows)
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            int kg = (int)(t0 % p.G), buf = 0, nseg[2] = {0, 0};
            bool first = true;
#if defined(VK_TRACE) && VK_TRACE == 6
            long long tr[4] = {0, 0, 0, 0};
            const long long tr_start = clock64();
#endif
            for (int i = 0; i < n; i++) {
                const int s = i % kTaSlots;
                const uint32_t ph = (uint32_t)((i / kTaSlots) & 1);
                TA_T(m0);
                TA_T(m1);
                if (!mbar_wait(&bready[s], ph)) { s_fail = 1; break; }
                TA_T(m2);
                if (first && nseg[buf] > 0 && !mbar_wait(&dfree[buf], (uint32_t)((nseg[buf] - 1) & 1))) { s_fail = 1; break; }
                TA_T(m3);
                TA_ACC(0, m0, m1); TA_ACC(1, m1, m2); TA_ACC(2, m2, m3);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a0 = smem_u32(slots + (size_t)s * kTaSlotBytes);
                const uint32_t b0 = a0 + kTaXBytes;
#ifndef VK_TA_EXP
#define VK_TA_EXP 0
#endif
#pragma unroll
                for (int kk = 0; kk < 4; kk++) {   // K = 16 per instruction = two 16-byte units along K
#if VK_TA_EXP == 2
                    continue;                       // (timing experiment: no MMA)
#endif
                    const uint64_t da = umma_desc(a0 + kk * 2 * Cfg::kLbo, Cfg::kLbo, 128);
                    const uint64_t db = umma_desc(b0 + kk * 2 * (kSBRows * 16), kSBRows * 16, 128);
                    const uint32_t accumulate = (first && kk == 0) ? 0u : 1u;
                    const uint32_t zero = 0u;
                    asm volatile(
                        "{\n\t"
                        ".reg .pred p;\n\t"
                        "setp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
                        "}\n" ::"r"(tmem + (uint32_t)(buf * 256)),
                        "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(zero)
                        : "memory");
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&sfree[s]))
                             : "memory");
                first = false;
#if defined(VK_TRACE) && VK_TRACE == 6
                { const long long m4 = clock64(); tr[3] += m4 - m3; }
#endif
                kg++;
                if (kg == p.G || i == n - 1) {   // the segment (one superblock's steps inside this CTA's range) ends
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                     smem_u32(&dready[buf]))
                                 : "memory");
                    nseg[buf]++;
                    buf ^= 1;
                    first = true;
                    if (kg == p.G) kg = 0;
                }
            }
#if defined(VK_TRACE) && VK_TRACE == 6
            long long* o = g_vk_trace + (blockIdx.x & 4095) * 16;
            o[8] = tr[0]; o[9] = tr[1]; o[10] = tr[2]; o[11] = tr[3]; o[12] = clock64() - tr_start; o[13] = n;
#endif
        }
    } else if (MR == 16 ? (warp == 0 || warp == 4) : (warp >= 4 && warp < 8)) {
        // ---------------------------------------------------------------- drain (a warp reads the lane quarter warp % 4)
        pdl_wait();
        const int dw = MR == 16 ? (warp >> 2) : (warp - 4);         // drain warp index
        const int dtid = dw * 32 + lane;
        const int m = MR == 16 ? lane : dw * 32 + lane;             // activation row held by this thread
        const int ncols = MR == 16 ? 128 : 256, col0 = MR == 16 ? dw * 128 : 0;   // accumulator columns this warp takes
        int sb = (int)(t0 / p.G), kg0 = (int)(t0 % p.G);
        int buf = 0, nseg[2] = {0, 0};
        bool ok = true;
        // rows [r0, r1) of superblock fsb: the nc partial slabs added in slab order, rounded, stored
        auto add_partials = [&](int fsb, int nc, int r0, int r1) {
            constexpr int V4 = kPS / 4;   // float4 columns of a partial row
            for (int item = dtid; item < (r1 - r0) * V4; item += kDrainThreads) {
                const int r = r0 + item / V4, v = item % V4;
                const int nrow = fsb * kSBRows + r;
                const float4* src = reinterpret_cast<const float4*>(p.part + ((size_t)fsb * p.maxc * kSBRows + r) * kPS) + v;
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int c0 = 0; c0 < nc; c0 += 8) {
                    float4 b8[8];
#pragma unroll
                    for (int u = 0; u < 8; u++)
                        b8[u] = (c0 + u < nc) ? __ldcg(src + (size_t)(c0 + u) * kSBRows * V4) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        if (c0 + u < nc) { sum.x += b8[u].x; sum.y += b8[u].y; sum.z += b8[u].z; sum.w += b8[u].w; }
                    }
                }
                if (nrow < p.N) {
                    const float o4[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
                    for (int e = 0; e < 4; e++)
                        if (4 * v + e < p.M) p.y[(size_t)(4 * v + e) * p.ldy + nrow] = f2bf(o4[e]);
                }
            }
        };
        for (int done = 0; done < n && ok;) {
            const int kga = kg0, kgb = (p.G - kg0 < n - done) ? p.G : kg0 + (n - done);
            const bool whole = (kga == 0 && kgb == p.G);
            const long long s0 = (long long)sb * p.G;
            const int c_first = p.S > 0 ? sb * p.S : step_owner(s0, p.T, p.P);
            if (!mbar_wait(&dready[buf], (uint32_t)(nseg[buf] & 1))) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float* pdst = p.part + (((size_t)sb * p.maxc + (blockIdx.x - c_first)) * kSBRows) * kPS;
#pragma unroll 1
            for (int c = 0; c < ncols / 32; c++) {
                uint32_t d[32];
                const int col = col0 + c * 32;
                const uint32_t taddr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(buf * 256 + col);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]), "=r"(d[8]),
                      "=r"(d[9]), "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15]), "=r"(d[16]),
                      "=r"(d[17]), "=r"(d[18]), "=r"(d[19]), "=r"(d[20]), "=r"(d[21]), "=r"(d[22]), "=r"(d[23]), "=r"(d[24]),
                      "=r"(d[25]), "=r"(d[26]), "=r"(d[27]), "=r"(d[28]), "=r"(d[29]), "=r"(d[30]), "=r"(d[31])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (m < p.M) {
                    if (whole) {
                        const size_t yoff = (size_t)m * p.ldy + (size_t)sb * kSBRows + col;
                        __nv_bfloat16* yrow = p.y + yoff;
                        const int lim = p.N - (sb * kSBRows + col);   // columns of this piece that exist
                        if (lim >= 32 && (yoff & 7) == 0) {
#pragma unroll
                            for (int e = 0; e < 32; e += 8) {
                                uint4 o;
                                o.x = pack_bf2(__uint_as_float(d[e]), __uint_as_float(d[e + 1]));
                                o.y = pack_bf2(__uint_as_float(d[e + 2]), __uint_as_float(d[e + 3]));
                                o.z = pack_bf2(__uint_as_float(d[e + 4]), __uint_as_float(d[e + 5]));
                                o.w = pack_bf2(__uint_as_float(d[e + 6]), __uint_as_float(d[e + 7]));
                                *reinterpret_cast<uint4*>(yrow + e) = o;
                            }
                        } else {
#pragma unroll
                            for (int e = 0; e < 32; e++)
                                if (e < lim) yrow[e] = f2bf(__uint_as_float(d[e]));
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; e++) __stcg(pdst + (size_t)(col + e) * kPS + m, __uint_as_float(d[e]));
                    }
                } else if (!whole && m < kPS) {   // rows M.. of a slab are read by the final addition: keep them defined
#pragma unroll
                    for (int e = 0; e < 32; e++) __stcg(pdst + (size_t)(col + e) * kPS + m, 0.f);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&dfree[buf]);
            nseg[buf]++;
            buf ^= 1;
            if (!whole) {
                ta_drain_sync<kDrainThreads>();
                if (p.S > 0) {
                    // aligned mode: the S CTAs of this superblock started together with equal shares of K. Each has stored
                    // its partial sums, waits (bounded) for the others, then adds up its own share of the rows in slice order.
                    const int nc = p.S, slot = blockIdx.x - c_first;
                    int* arrive = p.counters + sb;
                    int* depart = p.counters + 2048 + sb;
                    if (dtid == 0) {
                        __threadfence();
                        atomicAdd(arrive, 1);
                        int seen = 0;
                        for (uint32_t it = 0; it < (1u << 20); it++) {
                            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(arrive) : "memory");
                            if (seen >= nc) break;
                            __nanosleep(32);
                        }
                        s_last = seen >= nc;
                        if (!s_last) vk_set_status(VK_ST_FLAG_TIMEOUT);
                    }
                    ta_drain_sync<kDrainThreads>();
                    if (s_last) add_partials(sb, nc, slot * kSBRows / nc, (slot + 1) * kSBRows / nc);
                    ta_drain_sync<kDrainThreads>();
                    if (dtid == 0) {
                        const int old = atomicAdd(depart, 1);
                        if (old == nc - 1) { *arrive = 0; *depart = 0; __threadfence(); }
                    }
                } else {
                    if (dtid == 0) {   // the CTA that arrives last adds up the partial sums of all ranges, in range order
                        __threadfence();
                        const int ncontrib = step_owner(s0 + p.G - 1, p.T, p.P) - c_first + 1;
                        const int old = atomicAdd(&p.counters[sb], 1);
                        s_last = (old == ncontrib - 1) ? ncontrib : 0;
                        if (s_last) p.counters[sb] = 0;
                    }
                    ta_drain_sync<kDrainThreads>();
                    const int ncontrib = s_last;
                    if (ncontrib) {
                        __threadfence();
                        add_partials(sb, ncontrib, 0, kSBRows);
                    }
                    ta_drain_sync<kDrainThreads>();   // s_last is reused by the next segment
                }
            }
            done += kgb - kga;
            kg0 = 0;
            sb++;
        }
        if (!ok) s_fail = 1;
    } else {
        // ---------------------------------------------------------------- expansion (warps 3, 5..19): weights only
        const int cw = MR == 16 ? (warp == 3 ? 0 : warp - 4) : (warp == 0 ? 0 : warp == 3 ? 1 : warp - 6);   // 0..15
        const int g = lane >> 2, t = lane & 3;
        // Two groups of eight warps take alternate steps (a warp expands a whole 32-row chunk of its steps): the waits of
        // one group (weights landed, slot free, stores visible) hide behind the other group's arithmetic.
        const int grp = cw >> 3, ej = cw & 7;
        bool waited = false;
        const __nv_bfloat162 k128 = __halves2bfloat162(__ushort_as_bfloat16((unsigned short)0x4300u),
                                                       __ushort_as_bfloat16((unsigned short)0x4300u));
#if defined(VK_TRACE) && VK_TRACE == 6
        long long tr[4] = {0, 0, 0, 0};
        const long long tr_start = clock64();
#endif
        for (int i = grp; i < n; i += 2) {
            const int st = i % kTaStages;
            TA_T(c0);
            if (!mbar_wait(&wfull[st], (uint32_t)((i / kTaStages) & 1))) { s_fail = 1; break; }
            TA_T(c1);
            const uint8_t* stage = smem + (size_t)st * kTaWBytes;
            const uint4 wv0 = *reinterpret_cast<const uint4*>(stage + ej * kChunkBytes + lane * 16);
            const uint4 wv1 = *reinterpret_cast<const uint4*>(stage + ej * kChunkBytes + 512 + lane * 16);
            const uint4 sbp = *reinterpret_cast<const uint4*>(stage + ej * kChunkBytes + 1024 + g * 16);
            __syncwarp();
            if (lane == 0) mbar_arrive(&wempty[st]);   // this warp's codes and scale words are in registers
            const int s = i % kTaSlots;
            // (the first slots need no wait; from here on progress depends on the kernel in front, through the x records:
            // wait for it here rather than in the bounded poll below)
            if (i >= kTaSlots && !waited) { pdl_wait(); waited = true; }
            TA_T(c2);
            if (i >= kTaSlots && !mbar_wait(&sfree[s], (uint32_t)((i / kTaSlots - 1) & 1))) { s_fail = 1; break; }
            TA_T(c3);
            const uint32_t sbw[4] = {sbp.x, sbp.y, sbp.z, sbp.w};   // (scale | bias) of rows g, g + 8 of stripe 0, of stripe 1
            uint8_t* brow0 = slots + (size_t)s * kTaSlotBytes + kTaXBytes + (size_t)(32 * ej + g) * 16 + 4 * t;
#pragma unroll
            for (int es = 0; es < 2; es++) {
#if VK_TA_EXP == 1
                if (sbw[0] != 0x12345678u) continue;   // (timing experiment: no expansion, no stores)
#endif
                __nv_bfloat162 s2[2], b2[2];   // each doubled into a bf16 pair
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    uint32_t v = __byte_perm(sbw[2 * es + h], 0, 0x1010);
                    s2[h] = *reinterpret_cast<__nv_bfloat162*>(&v);
                    v = __byte_perm(sbw[2 * es + h], 0, 0x3232);
                    b2[h] = *reinterpret_cast<__nv_bfloat162*>(&v);
                }
                const uint32_t wq[4] = {es ? wv1.x : wv0.x, es ? wv1.y : wv0.y, es ? wv1.z : wv0.z, es ? wv1.w : wv0.w};
                uint8_t* brow = brow0 + es * 256;
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    uint32_t a[4];
                    unpack_codes(wq[q], a);
                    // register r: row + 8 (r & 1), columns 16 q + 8 (r >> 1) + 2 t, + 1 -> unit 2 q + (r >> 1) along K
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        const __nv_bfloat162 u2 = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&a[r]), k128);   // exact: 0..15
                        const __nv_bfloat162 w2 = __hfma2(u2, s2[r & 1], b2[r & 1]);                          // one rounding
                        *reinterpret_cast<__nv_bfloat162*>(brow + (size_t)(2 * q + (r >> 1)) * (kSBRows * 16) + (r & 1) * 128) = w2;
                    }
                }
            }
            TA_T(c4);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> visible to the MMA
            __syncwarp();
            if (lane == 0) mbar_arrive(&bready[s]);
            TA_T(c5);
            TA_ACC(0, c0, c1); TA_ACC(1, c2, c3); TA_ACC(2, c3, c4); TA_ACC(3, c4, c5);
        }
#if defined(VK_TRACE) && VK_TRACE == 6
        if (cw == 0 && lane == 0) {
            long long* o = g_vk_trace + (blockIdx.x & 4095) * 16;
            for (int u = 0; u < 4; u++) o[u] = tr[u];
            o[4] = clock64() - tr_start;
        }
#endif
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 2) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
    if (threadIdx.x == 0 && s_fail) vk_set_status(VK_ST_MBAR_TIMEOUT);
}

// p: filled for w4_plan(N, K, 1) (one CTA per SM); rows128: p.xrec holds 16 KB activation tiles (up to 128 rows) and the
// partial-sum slabs are 128 floats wide, else x records (up to 16 rows) and 16-float slabs
template <int MR>
static cudaError_t w4_tacc_launch_t(const W4Params& p, cudaStream_t stream) {
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!configured[dev].load(std::memory_order_acquire)) {
        e = cudaFuncSetAttribute(w4_tacc_kernel<MR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TaCfg<MR>::kSmem);
        if (e != cudaSuccess) return e;
        configured[dev].store(true, std::memory_order_release);
    }
    return vk_launch(w4_tacc_kernel<MR>, dim3(p.P), dim3(TaCfg<MR>::kThreads), TaCfg<MR>::kSmem, stream, p);
}
cudaError_t w4_tacc_launch(const W4Params& p, cudaStream_t stream) { return w4_tacc_launch_t<16>(p, stream); }
cudaError_t w4_tacc_launch128(const W4Params& p, cudaStream_t stream) { return w4_tacc_launch_t<128>(p, stream); }

}  // namespace
