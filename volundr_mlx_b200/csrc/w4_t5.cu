// The INT4 small-M GEMM (1..16 activation rows) with the product on the 5th-generation tensor cores: the same
// arithmetic, work split and result as w4_gemm_kernel<MT, 0> (acc += s * (x_g . u_g) + b * sum(x_g) per 64-column group,
// see w4_gemm.cu), but x_g . (128 + u_g) is formed by tcgen05.mma instead of mma.sync.
//
// Why: at 16 rows the mma.sync kernel is bound by the warps' own instruction stream (188 instructions per 1152-byte
// chunk, sixteen of them m16n8k16 at one per 8 cycles and scheduler on this architecture, a quarter of the tcgen05
// rate, 56 of them the logic operations that expand the codes). tcgen05.mma is issued by ONE thread for the whole CTA
// and runs beside the warps, which are left with the expansion and two fused multiply-adds per output and group.
//
// One CTA per SM, 18 warps:
//   warp 0        one lane: the TMA producer of w4_gemm_kernel (9216-byte weight step + the group's x record per
//                 stage, the weights before the dependency wait, an 8-stage ring)
//   warp 1        one lane: per step, waits for the expanded weights and the x record and issues 8 tcgen05.mma
//                 (2 tiles of 128 weight rows as the M side, the 16 activation rows as N, K = 16 each), D = one of four
//                 32-column slots of tensor memory, then commits them to the slot's "ready" barrier
//   warps 2..17   (a) expand the codes of their 16 rows x 64 columns of the step to bf16 128 + u (the lop3 of the
//                 mma.sync kernel) and store them as the A operand, K-major without swizzle: [column / 8][row 256][8];
//                 (b) one step later, read their 32 weight rows x 8 activation rows of the step's D from tensor memory
//                 and add s * D + (b - 128 s) * S to their fp32 accumulators (one weight row per thread).
// The x record is the B operand as it lies in the stage ([column / 8][row 16][8], see xrec.cuh). A-operand slots rotate
// over three buffers: a warp writes slot i mod 3 only after it has consumed step i - 3's D, i.e. after those MMAs have
// finished reading the slot. Range ends, partial sums and the final additions are those of w4_gemm_kernel (same
// workspace layout, same fixed order). Every wait is bounded; a wait that runs out sets the status word and the CTA
// winds down (tensor memory is freed on every path).
#include <atomic>

#include "common.cuh"

namespace {

constexpr int kT5Warps = 16;                          // expansion / accumulation warps
constexpr int kT5Threads = 32 * (2 + kT5Warps);       // 576
constexpr int kT5WBytes = kBlocksPerSB * kChunkBytes;   // 9216: one step of packed weights
constexpr int kT5ABytes = kSBRows * 64 * 2;             // 32 KB: [8][256][8] bf16
constexpr int kT5DSlots = 8;                            // 8 x 32 columns of tensor memory
constexpr int kT5XSlots = 12;                           // ring of x records
// LAG = steps between a warp's expansion of a step and its accumulation of the same step: the round trip "last warp has
// stored -> the MMA thread wakes and issues -> the MMAs finish -> the commit arrives -> the warps wake" takes about a
// microsecond, two to three steps' worth of work, and a warp that waited for it after every step would run at that
// latency. Weight stages are released as soon as the codes are in registers (the whole ring stays in flight towards
// HBM); the x records have a ring of their own and stay until the step's accumulation has read the group sums.
template <int LAG> struct T5Cfg {
    static constexpr int kASlots = LAG + 1;           // slot of step i is rewritten at step i + LAG + 1, after step i's D was read
    static constexpr int kStages = LAG >= 3 ? 7 : 10;
    static constexpr int kBars = 2 * kStages + 2 * kT5XSlots + kASlots + 2 * kT5DSlots;
    static constexpr size_t kXOff = (size_t)kStages * kT5WBytes;
    static constexpr size_t kAOff = ((kXOff + (size_t)kT5XSlots * kXRecBytes + 127) / 128) * 128;
    static constexpr size_t kBarOff = kAOff + (size_t)kASlots * kT5ABytes;
    static constexpr size_t kSmem = kBarOff + kBars * 8;
    static_assert(kSmem <= 227 * 1024, "does not fit a CTA's shared memory");
    static_assert(kT5DSlots > LAG && kT5XSlots > LAG + 1, "a slot must have been read before it is written again");
};

#if defined(VK_TRACE) && VK_TRACE == 5
#define T5_T(var) const long long var = clock64()
#define T5_ACC(slot, a, b) tr[slot] += (b) - (a)
#else
#define T5_T(var) do { } while (0)
#define T5_ACC(slot, a, b) do { } while (0)
#endif

__device__ __forceinline__ void t5_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }

template <int LAG>
__global__ void __launch_bounds__(kT5Threads, 1) w4_t5_kernel(const W4Params p) {
    extern __shared__ __align__(128) uint8_t smem[];
    using Cfg = T5Cfg<LAG>;
    constexpr int kT5Stages = Cfg::kStages, kT5ASlots = Cfg::kASlots;
    uint8_t* xring = smem + Cfg::kXOff;
    uint8_t* abuf = smem + Cfg::kAOff;
    uint64_t* wfull = reinterpret_cast<uint64_t*>(smem + Cfg::kBarOff);
    uint64_t* wempty = wfull + kT5Stages;      // every warp has its codes of the stage in registers
    uint64_t* xfull = wempty + kT5Stages;
    uint64_t* xempty = xfull + kT5XSlots;      // every warp has read the record's group sums (after its MMAs finished)
    uint64_t* aready = xempty + kT5XSlots;     // [A slot] the step's expanded weights are in place
    uint64_t* dready = aready + kT5ASlots;     // [D slot] the step's MMAs have finished
    uint64_t* dfree = dready + kT5DSlots;      // [D slot] every accumulation warp has read the slot
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
        for (int s = 0; s < kT5Stages; s++) {
            mbar_init(&wfull[s], 1);
            mbar_init(&wempty[s], kT5Warps);
        }
        for (int s = 0; s < kT5XSlots; s++) {
            mbar_init(&xfull[s], 1);
            mbar_init(&xempty[s], kT5Warps);
        }
        for (int s = 0; s < kT5ASlots; s++) mbar_init(&aready[s], kT5Warps);
        for (int s = 0; s < kT5DSlots; s++) {
            mbar_init(&dready[s], 1);
            mbar_init(&dfree[s], kT5Warps);
        }
        mbar_fence_init();
        s_fail = 0;
    }
    if (warp == 1) {   // kT5DSlots x 32 columns of tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)),
                     "r"((uint32_t)(32 * kT5DSlots))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    if (warp == 0) {
        // ---------------------------------------------------------------- producers: lane 0 weights, lane 1 x records
        if (lane == 0) {
            const uint8_t* wsrc = p.wp + (size_t)t0 * kT5WBytes;
            const int pre = n < kT5Stages ? n : kT5Stages;
            for (int i = 0; i < pre; i++) {   // weights depend on no earlier kernel
                mbar_expect_tx(&wfull[i], kT5WBytes);
                tma_bulk_g2s(smem + (size_t)i * kT5WBytes, wsrc + (size_t)i * kT5WBytes, kT5WBytes, &wfull[i]);
            }
            pdl_wait();
            pdl_launch_dependents();
            int ws = 0;
            uint32_t wpar = 0;
            const uint8_t* wnext = wsrc + (size_t)pre * kT5WBytes;
            for (int i = pre; i < n; i++) {   // the weights of step i go into the stage that step i - pre's codes have left
                if (!mbar_wait(&wempty[ws], wpar)) { s_fail = 1; break; }
                fence_proxy_async_smem();   // (the expansion warps read the codes with ld.shared)
                mbar_expect_tx(&wfull[ws], kT5WBytes);
                tma_bulk_g2s(smem + (size_t)ws * kT5WBytes, wnext, kT5WBytes, &wfull[ws]);
                wnext += kT5WBytes;
                if (++ws == kT5Stages) { ws = 0; wpar ^= 1u; }
            }
        } else if (lane == 1) {
            pdl_wait();   // the x records are the output of the kernel in front
            int kg = (int)(t0 % p.G);
            int xs = 0;
            uint32_t xpar = 0;
            for (int i = 0; i < n; i++) {
                if (i >= kT5XSlots && !mbar_wait(&xempty[xs], xpar)) { s_fail = 1; break; }
                fence_proxy_async_smem();   // (the warps read the group sums of a record with ld.shared)
                mbar_expect_tx(&xfull[xs], kXRecBytes);
                tma_bulk_g2s(xring + (size_t)xs * kXRecBytes, p.xrec + (size_t)kg * kXRecBytes, kXRecBytes, &xfull[xs]);
                kg = kg + 1 == p.G ? 0 : kg + 1;
                if (++xs == kT5XSlots) { xs = 0; if (i >= kT5XSlots) xpar ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0) {
            pdl_wait();
            // instruction descriptor: D fp32, A and B bf16, both K-major, N = 16 (activation rows), M = 128 (weight rows)
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(16 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
#if defined(VK_TRACE) && VK_TRACE == 5
            long long tr[4] = {0, 0, 0, 0};
            const long long tr_start = clock64();
#endif
            for (int i = 0; i < n; i++) {
                const int as = i % kT5ASlots, ds = i % kT5DSlots, xs = i % kT5XSlots;
                T5_T(m0);
                if (!mbar_wait(&xfull[xs], (uint32_t)((i / kT5XSlots) & 1))) { s_fail = 1; break; }
                T5_T(m1);
                if (!mbar_wait(&aready[as], (uint32_t)((i / kT5ASlots) & 1))) { s_fail = 1; break; }
                T5_T(m2);
                if (i >= kT5DSlots && !mbar_wait(&dfree[ds], (uint32_t)((i / kT5DSlots - 1) & 1))) { s_fail = 1; break; }
                T5_T(m3);
                T5_ACC(0, m0, m1); T5_ACC(1, m1, m2); T5_ACC(2, m2, m3);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a0 = smem_u32(abuf + (size_t)as * kT5ABytes);
                const uint32_t b0 = smem_u32(xring + (size_t)xs * kXRecBytes);
#ifndef VK_T5_EXP
#define VK_T5_EXP 0
#endif
#pragma unroll
                for (int it = 0; it < 8; it++) {   // K = 16 per instruction = two 16-byte units along K
#if VK_T5_EXP == 1
                    const int tile = it & 1, kk = it >> 1;      // the two tiles' accumulators alternate
#else
                    const int tile = it >> 2, kk = it & 3;
#endif
#if VK_T5_EXP == 2
                    if (tile == 1) continue;                    // (timing experiment: half the MMAs)
#elif VK_T5_EXP == 3
                    if (it > 0) continue;                       // (timing experiment: one MMA)
#endif
                    const uint64_t da = umma_desc(a0 + tile * 128 * 16 + kk * 2 * (kSBRows * 16), kSBRows * 16, 128);
                    const uint64_t db = umma_desc(b0 + kk * 2 * (16 * 16), 16 * 16, 128);
#if VK_T5_EXP == 4
                    const uint32_t accumulate = 0u;             // (timing experiment: no MMA depends on another)
#else
                    const uint32_t accumulate = kk > 0 ? 1u : 0u;
#endif
                    const uint32_t zero = 0u;
                    asm volatile(
                        "{\n\t"
                        ".reg .pred p;\n\t"
                        "setp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
                        "}\n" ::"r"(tmem + (uint32_t)(ds * 32 + tile * 16)),
                        "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(zero)
                        : "memory");
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&dready[ds]))
                             : "memory");
#if defined(VK_TRACE) && VK_TRACE == 5
                { const long long m4 = clock64(); tr[3] += m4 - m3; }
#endif
            }
#if defined(VK_TRACE) && VK_TRACE == 5
            long long* o = g_vk_trace + (blockIdx.x & 4095) * 16;
            o[8] = tr[0]; o[9] = tr[1]; o[10] = tr[2]; o[11] = tr[3]; o[12] = clock64() - tr_start;
#endif
        }
    } else {
        // ---------------------------------------------------------------- expansion + accumulation (warps 2..17)
        pdl_wait();
        const int cw = warp - 2;                 // 0..15
        const int ctid = threadIdx.x - 64;       // 0..511
        const int g = lane >> 2, t = lane & 3;
        // (a) this warp expands stripe es (16 rows) of chunk ej (32 rows) of every step
        const int ej = cw >> 1, es = cw & 1;
        // (b) and accumulates the weight rows of tensor-memory lanes 32 quarter .. (a warp may only read the quarter of
        // the lanes given by its index mod 4) of tile `tile`, activation rows 8 colset .. 8 colset + 7
        const int colset = cw >> 3, tile = (cw >> 2) & 1, quarter = warp & 3;
        const int R = tile * 128 + quarter * 32 + lane;                 // weight row inside the superblock
        const int sb_word = (R >> 5) * kChunkBytes + 1024 + (((lane & 7) << 2) + ((lane >> 4) << 1) + ((lane >> 3) & 1)) * 4;
        const bool live = colset * 8 < p.M;       // (up to 8 rows: the second column set has nothing to add)
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; e++) acc[e] = 0.f;
        int sb = (int)(t0 / p.G), kg = (int)(t0 % p.G);
        int seg_kg0 = kg;
        bool ok = true;

        auto zero_acc = [&]() {
#pragma unroll
            for (int e = 0; e < 8; e++) acc[e] = 0.f;
        };
        auto store_partial = [&](float* dst) {
            if (live) {
                float4* d4 = reinterpret_cast<float4*>(dst + (size_t)R * 16 + colset * 8);
                __stcg(d4, make_float4(acc[0], acc[1], acc[2], acc[3]));
                __stcg(d4 + 1, make_float4(acc[4], acc[5], acc[6], acc[7]));
            } else if (colset == 1) {   // rows 8..15 of a slab are read by the final addition: keep them defined
                float4* d4 = reinterpret_cast<float4*>(dst + (size_t)R * 16 + 8);
                __stcg(d4, make_float4(0.f, 0.f, 0.f, 0.f));
                __stcg(d4 + 1, make_float4(0.f, 0.f, 0.f, 0.f));
            }
        };
        // rows [r0, r1) of superblock fsb: the nc partial slabs added in slab order, rounded, stored
        auto add_partials = [&](int fsb, int nc, int r0, int r1) {
            constexpr int V4 = 4;   // float4 columns of a 16-float partial row
            for (int item = ctid; item < (r1 - r0) * V4; item += 512) {
                const int r = r0 + item / V4, v = item % V4;
                const int nrow = fsb * kSBRows + r;
                const float4* src = reinterpret_cast<const float4*>(p.part + ((size_t)fsb * p.maxc * kSBRows + r) * 16) + v;
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int c0 = 0; c0 < nc; c0 += 8) {
                    float4 buf[8];
#pragma unroll
                    for (int u = 0; u < 8; u++)
                        buf[u] = (c0 + u < nc) ? __ldcg(src + (size_t)(c0 + u) * kSBRows * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        if (c0 + u < nc) { sum.x += buf[u].x; sum.y += buf[u].y; sum.z += buf[u].z; sum.w += buf[u].w; }
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
        auto flush = [&](int fsb, int kga, int kgb) {
            const bool whole = (kga == 0 && kgb == p.G);
            const long long s0 = (long long)fsb * p.G;
            const int c_first = p.S > 0 ? fsb * p.S : step_owner(s0, p.T, p.P);
            if (whole) {
                const int nrow = fsb * kSBRows + R;
                if (live && nrow < p.N) {
#pragma unroll
                    for (int e = 0; e < 8; e++)
                        if (colset * 8 + e < p.M) p.y[(size_t)(colset * 8 + e) * p.ldy + nrow] = f2bf(acc[e]);
                }
            } else if (p.S > 0) {
                // aligned mode: the S CTAs of this superblock started together with equal shares of K. Each stores its
                // partial sums, waits (bounded) for the others, then adds up its own share of the rows in slice order.
                store_partial(p.part + (((size_t)fsb * p.maxc + (blockIdx.x - c_first)) * kSBRows) * 16);
                t5_sync();
                const int nc = p.S, slot = blockIdx.x - c_first;
                int* arrive = p.counters + fsb;
                int* depart = p.counters + 2048 + fsb;
                if (ctid == 0) {
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
                t5_sync();
                if (s_last) add_partials(fsb, nc, slot * kSBRows / nc, (slot + 1) * kSBRows / nc);
                t5_sync();
                if (ctid == 0) {
                    const int old = atomicAdd(depart, 1);
                    if (old == nc - 1) { *arrive = 0; *depart = 0; __threadfence(); }
                }
            } else {
                store_partial(p.part + (((size_t)fsb * p.maxc + (blockIdx.x - c_first)) * kSBRows) * 16);
                t5_sync();
                if (ctid == 0) {   // the CTA that arrives last adds up the partial sums of all ranges, in range order
                    __threadfence();
                    const int ncontrib = step_owner(s0 + p.G - 1, p.T, p.P) - c_first + 1;
                    const int old = atomicAdd(&p.counters[fsb], 1);
                    s_last = (old == ncontrib - 1) ? ncontrib : 0;
                    if (s_last) p.counters[fsb] = 0;
                }
                t5_sync();
                const int ncontrib = s_last;
                if (ncontrib) {
                    __threadfence();
                    add_partials(fsb, ncontrib, 0, kSBRows);
                }
                t5_sync();   // s_last is reused by the next flush
            }
            zero_acc();
        };

        int st_d = 0;
        uint32_t ph_d = 0;
        uint32_t sbq[LAG + 1];   // (scale | bias) of this thread's weight row, steps i - LAG .. i (registers: shifted, not indexed)
#pragma unroll
        for (int u = 0; u <= LAG; u++) sbq[u] = 0u;
#if defined(VK_TRACE) && VK_TRACE == 5
        long long tr[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        const long long tr_start = clock64();
#endif
        for (int i = 0; i < n + LAG && ok; i++) {
#pragma unroll
            for (int u = 0; u < LAG; u++) sbq[u] = sbq[u + 1];
            if (i < n) {
                // ---- (a) expand this warp's 16 rows x 64 columns of step i into A slot i mod (LAG + 1)
                T5_T(c0);
                if (!mbar_wait(&wfull[st_d], ph_d)) { ok = false; break; }
                T5_T(c1);
                T5_ACC(0, c0, c1);
                const uint8_t* stage = smem + (size_t)st_d * kT5WBytes;
                const uint4 wv = *reinterpret_cast<const uint4*>(stage + ej * kChunkBytes + es * 512 + lane * 16);
                sbq[LAG] = *reinterpret_cast<const uint32_t*>(stage + sb_word);
                __syncwarp();
                if (lane == 0) mbar_arrive(&wempty[st_d]);   // this warp's codes and scale words are in registers
                const uint32_t wq[4] = {wv.x, wv.y, wv.z, wv.w};
                uint8_t* arow = abuf + (size_t)(i % kT5ASlots) * kT5ABytes + (size_t)(32 * ej + 16 * es + g) * 16 + 4 * t;
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    uint32_t a[4];
                    unpack_codes(wq[q], a);
                    // register r: row + 8 (r & 1), columns 16 q + 8 (r >> 1) + 2 t, + 1 -> unit 2 q + (r >> 1) along K
#pragma unroll
                    for (int r = 0; r < 4; r++)
                        *reinterpret_cast<uint32_t*>(arow + (size_t)(2 * q + (r >> 1)) * (kSBRows * 16) + (r & 1) * 128) = a[r];
                }
                T5_T(c2);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> visible to the MMA
                T5_T(c3);
                __syncwarp();
                if (lane == 0) mbar_arrive(&aready[i % kT5ASlots]);
                if (++st_d == kT5Stages) { st_d = 0; ph_d ^= 1u; }
                T5_T(c4);
                T5_ACC(1, c1, c2); T5_ACC(2, c2, c3); T5_ACC(3, c3, c4);
            }
            if (i >= LAG) {
                // ---- (b) step e = i - LAG: D from tensor memory, scale and bias term, into the accumulators
                const int e = i - LAG, ds = e % kT5DSlots;
                T5_T(e0);
                if (!mbar_wait(&dready[ds], (uint32_t)((e / kT5DSlots) & 1))) { ok = false; break; }
                T5_T(e1);
                T5_ACC(4, e0, e1);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t d[8];
                const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(ds * 32 + tile * 16 + colset * 8);
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                             : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7])
                             : "r"(taddr));
                const int xs = e % kT5XSlots;
                if (!mbar_wait(&xfull[xs], (uint32_t)((e / kT5XSlots) & 1))) { ok = false; break; }   // (long complete: the MMAs read it)
                const uint32_t sbw = sbq[0];
                const float4* sums = reinterpret_cast<const float4*>(xring + (size_t)xs * kXRecBytes + 2048 + colset * 32);
                const float4 x0 = sums[0], x1 = sums[1];
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                T5_T(e2);
                T5_ACC(5, e1, e2);
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&dfree[ds]);
                    mbar_arrive(&xempty[xs]);
                }
                const float sc = bf_lo(sbw), cb = fmaf(-128.f, sc, bf_hi(sbw));
                const float xsum[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                for (int c = 0; c < 8; c++) acc[c] = fmaf(cb, xsum[c], fmaf(sc, __uint_as_float(d[c]), acc[c]));
                if (++kg == p.G) {
                    flush(sb, seg_kg0, p.G);
                    kg = 0; seg_kg0 = 0; sb++;
                }
            }
        }
#if defined(VK_TRACE) && VK_TRACE == 5
        const long long tr_loop = clock64() - tr_start;
#endif
        if (ok && kg != seg_kg0) flush(sb, seg_kg0, kg);
        if (!ok) s_fail = 1;
#if defined(VK_TRACE) && VK_TRACE == 5
        if (threadIdx.x == 64) {
            long long* o = g_vk_trace + (blockIdx.x & 4095) * 16;
            for (int u = 0; u < 6; u++) o[u] = tr[u];
            o[6] = tr_loop; o[7] = clock64() - tr_start; o[13] = n;
        }
#endif
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)(32 * kT5DSlots)) : "memory");
    }
    if (threadIdx.x == 0 && s_fail) vk_set_status(VK_ST_MBAR_TIMEOUT);
}


// p: filled for w4_plan(N, K, 1) (one CTA per SM)
cudaError_t w4_t5_launch(const W4Params& p, cudaStream_t stream) {
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!configured[dev].load(std::memory_order_acquire)) {
        e = cudaFuncSetAttribute(w4_t5_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)T5Cfg<2>::kSmem);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(w4_t5_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)T5Cfg<3>::kSmem);
        if (e != cudaSuccess) return e;
        configured[dev].store(true, std::memory_order_release);
    }
    if (g_w4_t5 == 2) return vk_launch(w4_t5_kernel<2>, dim3(p.P), dim3(kT5Threads), T5Cfg<2>::kSmem, stream, p);
    return vk_launch(w4_t5_kernel<3>, dim3(p.P), dim3(kT5Threads), T5Cfg<3>::kSmem, stream, p);
}

}  // namespace
