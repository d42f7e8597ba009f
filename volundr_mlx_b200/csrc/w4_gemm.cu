// INT4 affine (group 64 / 128) weight GEMM for 1..16 activation rows: y[M,N] = x[M,K] . dequant(w)[N,K]^T.
//
// Replaces mx.quantized_matmul as called by every nn.QuantizedLinear of the reference (volundr.py:185-190, 377-386,
// 645-648) and the reference's small-M kernel qmm_nax_prepped (agens-mlx-bench/smallm/qmm_nax.py:28-139). Like that
// kernel it multiplies the raw 4-bit codes on the tensor cores and applies scale and bias per (row, group) to the
// fp32 group product, acc += s * (x_g . u_g) + b * sum(x_g), with the per-group activation sums prepared ahead of
// the product (the reference's prep_nax.prep, smallm/prep_nax.py:123-148).
//
// Weight layout. The reference layout (convert.py:7-14: u32 [N, K/8], nibble j of a word = element 8w + j, lowest
// first; bf16 scales / biases [N, K/G]) is repacked once at load time (vk_w4_repack) into 1152-byte chunks, one per
// (32 output rows, 64 input columns), stored [superblock of 256 rows][64-column group][8 chunks]:
//   bytes    0..1023  codes  [stripe 2][lane 32][kstep 4] u32 : for lane (g = lane / 4, t = lane % 4), stripe s,
//                     kstep q the word holds the mma.m16n8k16 A fragment of rows r0 = 16 s + g, r1 = r0 + 8 and
//                     columns c = 16 q + 2 t: nibbles {0: (r0,c) 4: (r0,c+1) 1: (r1,c) 5: (r1,c+1) 2: (r0,c+8)
//                     6: (r0,c+9) 3: (r1,c+8) 7: (r1,c+9)}, so (w >> 4 i) & 0x000F000F | 0x43004300 is fragment
//                     register i as two bf16 values 128 + u.
//   bytes 1024..1151  [g 8][4] u32 = (scale | bias << 16) of rows g, g + 8, 16 + g, 24 + g.
// One step of the kernel = one (superblock, group) = 9216 contiguous bytes, fetched by one TMA bulk copy; the packed
// size equals the algorithmic N*K/2 + N*(K/64)*4 bytes and no byte of it is read twice.
//
// Activation layout ("x records"). Per 64-column group one 2176-byte record: x[16 rows][64] bf16 stored
// [16-byte piece 8][row 16][8 bf16] (conflict-free ldmatrix; also a tcgen05 K-major operand), then the sixteen rows' sums over the
// group's 64 columns as fp32 (64 bytes; the record's last 64 bytes are unused). The kernel adds (bias - 128 scale) * S
// to the accumulator with them. vk_w4_gemm builds the records from a row-major x with a small kernel.
//
// Work split. total = superblocks * groups steps, in superblock-major order, dealt in equal contiguous ranges to
// P persistent CTAs (two per SM). A CTA is one producer warp (TMA into an 8-stage ring: weights as soon as the CTA
// starts, the x record once the kernel's predecessor has finished) and eight consumer warps, one 32-row block each.
// A range that does not cover a superblock's whole K writes fp32 partial sums; the CTA that arrives last at the
// superblock (arrival counter, left at zero) adds the partials in range order, so the result does not depend on
// scheduling and a row's result is the same for every M (the reference lists batch-variant matmuls as an open
// problem, NOTES_BATCHED_SERVE.md:256-258).
#include "common.cuh"
#include "xrec.cuh"

namespace {

constexpr int kBlocksPerSB = 8;                                 // 32-row blocks per superblock = consumer warps
constexpr int kSBRows = 32 * kBlocksPerSB;                      // 256
constexpr int kThreads = 32 * (1 + kBlocksPerSB);               // 288
constexpr size_t kCounterBytes = 16384;                         // arrival counters at the head of the workspace

// Weight formats the kernel streams. 0: 4-bit codes + (scale, bias), 1152-byte chunks. 1: plain bf16 (the linears the
// reference keeps unquantised, convert.py:16-17; the lm_head above all), 4096-byte chunks of 32 rows x 64 columns
// stored [stripe 2][kstep 4][lane 32][4 u32] = the mma A fragments as they are loaded.
template <int FMT> struct Fmt;
#ifndef VK_W4_STAGES
#define VK_W4_STAGES 8
#endif
#ifndef VK_W4_CTAS_PER_SM
#define VK_W4_CTAS_PER_SM 2
#endif
template <> struct Fmt<0> {
    static constexpr int kChunk = 1152, kStages = VK_W4_STAGES, kCtasPerSM = VK_W4_CTAS_PER_SM;
    static constexpr int kWStage = kBlocksPerSB * kChunk, kStage = kWStage + kXRecBytes + 16;  // + 16 zero bytes
};
template <> struct Fmt<1> {
    static constexpr int kChunk = 4096, kStages = 6, kCtasPerSM = 1;
    static constexpr int kWStage = kBlocksPerSB * kChunk, kStage = kWStage + kXRecBytes + 16;  // + 16 zero bytes
};
template <int FMT> constexpr int wstage_bytes() { return Fmt<FMT>::kWStage; }
// x records per group a kernel variant reads: 16 activation rows each (MT = n-tiles of 8 rows: 1, 2, 4 or 8)
template <int MT> __host__ __device__ constexpr int n_records() { return MT <= 2 ? 1 : MT / 2; }
template <int FMT, int MT = 2> __host__ __device__ constexpr int stage_bytes() { return Fmt<FMT>::kWStage + n_records<MT>() * kXRecBytes + 16; }
template <int FMT, int MT = 2> constexpr size_t smem_bytes() {
    return (size_t)Fmt<FMT>::kStages * stage_bytes<FMT, MT>() + 2 * Fmt<FMT>::kStages * 8;
}
template <int FMT, int MT> __host__ __device__ constexpr int ctas_per_sm() { return MT <= 2 ? Fmt<FMT>::kCtasPerSM : 1; }
constexpr int kChunkBytes = Fmt<0>::kChunk;

struct W4Params {
    const uint8_t* wp;      // packed weights
    const uint8_t* xrec;    // [G][records per group] x records
    __nv_bfloat16* y;       // [M, ldy]
    float* part;            // [NSB][maxc][256][16] partial sums
    int* counters;          // [NSB] zero between launches
    long long T;            // NSB * G steps
    int M, N, NSB, G, P, ldy, maxc;
    int S;                  // > 0: aligned mode, CTA c = (superblock c / S, K slice c % S); 0: contiguous ranges
    int pf;                 // steps per CTA (beyond the ring) whose weights are prefetched into L2 before the wait for x
};

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// mma with a zero accumulator input (first k-step of a group)
__device__ __forceinline__ void mma_bf16_z(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
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

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// the CTA whose range [c T / P, (c + 1) T / P) holds step t
__device__ __forceinline__ int step_owner(long long t, long long T, int P) { return (int)(((t + 1) * P - 1) / T); }

template <int MT, int FMT>
__global__ void __launch_bounds__(kThreads, ctas_per_sm<FMT, MT>()) w4_gemm_kernel(const W4Params p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int MR = MT * 8;
    constexpr int PS = MR < 16 ? 16 : MR;                  // floats per row of a partial-sum slab
    constexpr int kXR = n_records<MT>() * kXRecBytes;      // bytes of x records per stage
    constexpr int kStages = Fmt<FMT>::kStages;
    constexpr int kStageBytes = stage_bytes<FMT, MT>();
    constexpr int kWStageBytes = Fmt<FMT>::kWStage;
    constexpr int kChunkB = Fmt<FMT>::kChunk;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)kStages * kStageBytes);
    uint64_t* empty = full + kStages;
    __shared__ int s_last;
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
        for (int s = 0; s < kStages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kBlocksPerSB);
        }
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        const uint8_t* wsrc = p.wp + (size_t)t0 * kWStageBytes;
        const int pre = n < kStages ? n : kStages;
        if (lane == 0) {
            // the weights depend on no earlier kernel: start streaming before waiting for the producer of x
            for (int i = 0; i < pre; i++) {
                mbar_expect_tx(&full[i], kWStageBytes + kXR);
                tma_bulk_g2s(smem + (size_t)i * kStageBytes, wsrc + (size_t)i * kWStageBytes, kWStageBytes, &full[i]);
            }
        }
        __syncwarp();
        {   // ... and pull the next steps of this CTA's range into L2 while the kernel before this one still runs: the
            // memory system is otherwise idle then, and the ring later fills from L2 instead of HBM
            const int pf_end = n < pre + p.pf ? n : pre + p.pf;
            for (int i = pre + lane; i < pf_end; i += 32)
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(wsrc + (size_t)i * kWStageBytes), "r"(kWStageBytes)
                             : "memory");
        }
        if (lane == 0) {
            pdl_wait();
            pdl_launch_dependents();
            // (running group index, stage and parity: this one thread feeds the whole CTA, so its loop carries no
            // division and no 64-bit arithmetic)
            int kg = (int)(t0 % p.G);
            for (int i = 0; i < pre; i++) {
                tma_bulk_g2s(smem + (size_t)i * kStageBytes + kWStageBytes, p.xrec + (size_t)kg * kXR, kXR, &full[i]);
                kg = kg + 1 == p.G ? 0 : kg + 1;
            }
            int st = 0;
            uint32_t par = 0;   // parity of the "empty" phase awaited next for stage st
            const uint8_t* wnext = wsrc + (size_t)pre * kWStageBytes;
#if defined(VK_TRACE) && VK_TRACE == 2
            long long tr_wait = 0, tr_t0 = clock64();
#endif
            for (int i = pre; i < n; i++) {
#if defined(VK_TRACE) && VK_TRACE == 2
                const long long tr_a = clock64();
#endif
                if (!mbar_wait(&empty[st], par)) break;
#if defined(VK_TRACE) && VK_TRACE == 2
                tr_wait += clock64() - tr_a;
#endif
                // (the consumers read the stage with ld.shared / ldmatrix, the refill writes it through the async proxy)
                fence_proxy_async_smem();
                uint8_t* dst = smem + (size_t)st * kStageBytes;
                mbar_expect_tx(&full[st], kWStageBytes + kXR);
                tma_bulk_g2s(dst, wnext, kWStageBytes, &full[st]);
                tma_bulk_g2s(dst + kWStageBytes, p.xrec + (size_t)kg * kXR, kXR, &full[st]);
                wnext += kWStageBytes;
                kg = kg + 1 == p.G ? 0 : kg + 1;
                if (++st == kStages) { st = 0; par ^= 1u; }
            }
#if defined(VK_TRACE) && VK_TRACE == 2
            g_vk_trace[(blockIdx.x & 4095) * 16 + 0] = tr_wait;            // producer: cycles waiting for a free stage
            g_vk_trace[(blockIdx.x & 4095) * 16 + 1] = clock64() - tr_t0;  // producer: cycles in the refill loop
            g_vk_trace[(blockIdx.x & 4095) * 16 + 2] = n;
#endif
        }
        return;
    }

    // -------------------------------------------------------------------- consumers
    // (nothing to do before the kernel in front has finished: wait for it here rather than in the bounded polls on the
    // first stage, which must not run out while that kernel is, say, legitimately waiting for a peer GPU)
    pdl_wait();
    const int j = warp - 1;                    // 32-row block inside the superblock
    const int g = lane >> 2, t = lane & 3;
    const int ctid = threadIdx.x - 32;         // 0..255
    float acc[2][MT][4];
#pragma unroll
    for (int s = 0; s < 2; s++)
#pragma unroll
        for (int jj = 0; jj < MT; jj++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[s][jj][e] = 0.f;

    // ldmatrix source of this lane inside an x record: row, and which 16-byte piece of each 32-byte k-step
    const int lm_mat = lane >> 3, lm_r = lane & 7;
    const int lm_row = (MT >= 2 ? (lm_mat >> 1) * 8 : 0) + lm_r;
    const int lm_half = lm_mat & 1;

    int sb = (int)(t0 / p.G), kg = (int)(t0 % p.G);
    int seg_kg0 = kg;
    bool ok = true;

    auto flush = [&](int fsb, int kga, int kgb) {
        const bool whole = (kga == 0 && kgb == p.G);
        const long long s0 = (long long)fsb * p.G;
        const int c_first = p.S > 0 ? fsb * p.S : step_owner(s0, p.T, p.P);
        if (!whole && p.S > 0) {
            // ---- aligned mode: the S CTAs of this superblock started together with equal shares of K. Each stores its
            // partial sums, waits (bounded) for the other S - 1, then adds up its own 256 / S rows in slice order.
            float* dst = p.part + (((size_t)fsb * p.maxc + (blockIdx.x - c_first)) * kSBRows) * PS;
#pragma unroll
            for (int s = 0; s < 2; s++)
#pragma unroll
                for (int jj = 0; jj < MT; jj++)
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const int r = j * 32 + s * 16 + g + h * 8;
                        __stcg(reinterpret_cast<float2*>(dst + (size_t)r * PS + jj * 8 + 2 * t),
                               make_float2(acc[s][jj][2 * h], acc[s][jj][2 * h + 1]));
                    }
            consumer_sync();
            const int nc = p.S, slot = blockIdx.x - c_first;
            int* arrive = p.counters + fsb;
            int* depart = p.counters + 2048 + fsb;
            if (ctid == 0) {
                __threadfence();   // after the barrier: orders every consumer's partial stores before the arrival
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
            consumer_sync();
            if (s_last) {   // (thread 0's acquire loads and the barrier order the partial sums before the reads below)
                constexpr int V4 = MR / 4;
                const int r0 = slot * kSBRows / nc, r1 = (slot + 1) * kSBRows / nc;
                for (int item = ctid; item < (r1 - r0) * V4; item += 256) {
                    const int r = r0 + item / V4, v = item % V4;
                    const int nrow = fsb * kSBRows + r;
                    const float4* src = reinterpret_cast<const float4*>(p.part + ((size_t)fsb * p.maxc * kSBRows + r) * PS) + v;
                    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int c0 = 0; c0 < nc; c0 += 8) {
                        float4 buf[8];
#pragma unroll
                        for (int u = 0; u < 8; u++)
                            buf[u] = (c0 + u < nc) ? __ldcg(src + (size_t)(c0 + u) * kSBRows * (PS / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
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
            }
            consumer_sync();
            if (ctid == 0) {   // the last one to leave puts both counters back to zero for the next launch
                const int old = atomicAdd(depart, 1);
                if (old == nc - 1) { *arrive = 0; *depart = 0; __threadfence(); }
            }
        } else if (!whole) {
            float* dst = p.part + (((size_t)fsb * p.maxc + (blockIdx.x - c_first)) * kSBRows) * PS;
#pragma unroll
            for (int s = 0; s < 2; s++)
#pragma unroll
                for (int jj = 0; jj < MT; jj++)
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const int r = j * 32 + s * 16 + g + h * 8;
                        __stcg(reinterpret_cast<float2*>(dst + (size_t)r * PS + jj * 8 + 2 * t),
                               make_float2(acc[s][jj][2 * h], acc[s][jj][2 * h + 1]));
                    }
            consumer_sync();
            // The CTA that arrives last at this superblock adds up the partial sums of all its ranges, in range order.
            // (Nobody waits: a wait for the other ranges would chain every CTA to its predecessor, whose last range
            // ends where this one's first begins.)
            if (ctid == 0) {
                __threadfence();   // after the barrier: orders every consumer's partial stores before the arrival
                const int ncontrib = step_owner(s0 + p.G - 1, p.T, p.P) - c_first + 1;
                const int old = atomicAdd(&p.counters[fsb], 1);
                s_last = (old == ncontrib - 1) ? ncontrib : 0;
                if (s_last) p.counters[fsb] = 0;  // ready for the next launch
            }
            consumer_sync();
            const int ncontrib = s_last;
            if (ncontrib) {
                __threadfence();
                constexpr int V4 = MR / 4;                                 // float4 columns of a partial row
                for (int item = ctid; item < kSBRows * V4; item += 256) {
                    const int r = item / V4, v = item % V4;
                    const int nrow = fsb * kSBRows + r;
                    const float4* src = reinterpret_cast<const float4*>(p.part + ((size_t)fsb * p.maxc * kSBRows + r) * PS) + v;
                    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int c0 = 0; c0 < ncontrib; c0 += 8) {             // eight loads in flight, added in range order
                        float4 buf[8];
#pragma unroll
                        for (int u = 0; u < 8; u++)
                            buf[u] = (c0 + u < ncontrib) ? __ldcg(src + (size_t)(c0 + u) * kSBRows * (PS / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (int u = 0; u < 8; u++) {
                            if (c0 + u < ncontrib) { sum.x += buf[u].x; sum.y += buf[u].y; sum.z += buf[u].z; sum.w += buf[u].w; }
                        }
                    }
                    if (nrow < p.N) {
                        const float o4[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
                        for (int e = 0; e < 4; e++)
                            if (4 * v + e < p.M) p.y[(size_t)(4 * v + e) * p.ldy + nrow] = f2bf(o4[e]);
                    }
                }
            }
            consumer_sync();  // s_last is reused by the next flush
        } else {
#pragma unroll
            for (int s = 0; s < 2; s++)
#pragma unroll
                for (int jj = 0; jj < MT; jj++)
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const int nrow = fsb * kSBRows + j * 32 + s * 16 + g + h * 8;
                        const int m = jj * 8 + 2 * t;
                        if (nrow < p.N) {
                            if (m < p.M) p.y[(size_t)m * p.ldy + nrow] = f2bf(acc[s][jj][2 * h]);
                            if (m + 1 < p.M) p.y[(size_t)(m + 1) * p.ldy + nrow] = f2bf(acc[s][jj][2 * h + 1]);
                        }
                    }
        }
#pragma unroll
        for (int s = 0; s < 2; s++)
#pragma unroll
            for (int jj = 0; jj < MT; jj++)
#pragma unroll
                for (int e = 0; e < 4; e++) acc[s][jj][e] = 0.f;
    };

    // per-lane offsets inside a stage that do not change from step to step: the four ldmatrix sources and the group
    // sums of this lane's activation rows
    uint32_t lm_off[4];
#pragma unroll
    for (int q = 0; q < 4; q++) lm_off[q] = kWStageBytes + ((2 * q + lm_half) * 16 + lm_row) * 16;
    uint32_t sum_off[MT];   // the fp32 group sums of activation rows 8 jj + 2 t, 8 jj + 2 t + 1
#pragma unroll
    for (int jj = 0; jj < MT; jj++) sum_off[jj] = kWStageBytes + (jj >> 1) * kXRecBytes + 2048 + ((jj & 1) * 8 + 2 * t) * 4;
    int st = 0;
    uint32_t phase = 0;
#if defined(VK_TRACE) && VK_TRACE == 2
    long long tc_wait = 0, tc_t0 = clock64();
#endif
    for (int i = 0; i < n; i++, st = (st + 1 == kStages ? 0 : st + 1), phase ^= (st == 0)) {
#if defined(VK_TRACE) && VK_TRACE == 2
        const long long tc_a = clock64();
#endif
        if (!mbar_wait(&full[st], phase)) { ok = false; break; }
#if defined(VK_TRACE) && VK_TRACE == 2
        tc_wait += clock64() - tc_a;
        if (i == 0 && threadIdx.x == 32) g_vk_trace[(blockIdx.x & 4095) * 16 + 5] = clock64() - tc_t0;   // first data
#endif
        const uint8_t* stage = smem + (size_t)st * kStageBytes;
        const uint8_t* ch = stage + j * kChunkB;
        const uint32_t stage_a = smem_u32(stage);
        if constexpr (FMT == 1) {
            static_assert(FMT == 0 || MT <= 2, "the bf16 format is built for up to 16 rows per pass");
            // plain bf16 weights: fragments as stored, accumulate straight into acc
#pragma unroll
            for (int q = 0; q < 4; q++) {
                uint32_t b[2 * MT];
                const uint32_t addr = stage_a + lm_off[q];
                if constexpr (MT == 2) {
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3])
                                 : "r"(addr));
                } else {
                    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(b[0]), "=r"(b[1]) : "r"(addr));
                }
#pragma unroll
                for (int s = 0; s < 2; s++) {
                    const uint4 av = *reinterpret_cast<const uint4*>(ch + ((s * 4 + q) * 32 + lane) * 16);
                    const uint32_t a[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
                    for (int jj = 0; jj < MT; jj++) mma_bf16(acc[s][jj], a, b[2 * jj], b[2 * jj + 1]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);
        } else {
        const uint4 w0 = *reinterpret_cast<const uint4*>(ch + lane * 16);
        const uint4 w1 = *reinterpret_cast<const uint4*>(ch + 512 + lane * 16);
        const uint4 sb4 = *reinterpret_cast<const uint4*>(ch + 1024 + g * 16);
        float d[2][MT][4];
        const uint32_t wq0[4] = {w0.x, w0.y, w0.z, w0.w};
        const uint32_t wq1[4] = {w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int q = 0; q < 4; q++) {
            uint32_t b[2 * MT];
            const uint32_t addr = stage_a + lm_off[q];
            if constexpr (MT >= 2) {
#pragma unroll
                for (int rec = 0; rec < n_records<MT>(); rec++)   // 16 activation rows per record
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(b[4 * rec]), "=r"(b[4 * rec + 1]), "=r"(b[4 * rec + 2]), "=r"(b[4 * rec + 3])
                                 : "r"(addr + rec * kXRecBytes));
            } else {
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(b[0]), "=r"(b[1]) : "r"(addr));
            }
            uint32_t a[4];
            unpack_codes(wq0[q], a);
#pragma unroll
            for (int jj = 0; jj < MT; jj++) {
                if (q == 0) mma_bf16_z(d[0][jj], a, b[2 * jj], b[2 * jj + 1]);
                else mma_bf16(d[0][jj], a, b[2 * jj], b[2 * jj + 1]);
            }
            unpack_codes(wq1[q], a);
#pragma unroll
            for (int jj = 0; jj < MT; jj++) {
                if (q == 0) mma_bf16_z(d[1][jj], a, b[2 * jj], b[2 * jj + 1]);
                else mma_bf16(d[1][jj], a, b[2 * jj], b[2 * jj + 1]);
            }
        }
        // group epilogue: acc += s * (D - 128 S) + b * S = s * D + (b - 128 s) * S, S = the group's sum of the activation
        // row in fp32 (written into the record by whoever produced it), two fused multiply-adds per accumulator. (An
        // earlier form sent the second term through one more mma per n-tile, with S split into two bf16 parts: at 16
        // rows the kernel is bound by the throughput of mma.sync itself, so four mma out of twenty were a fifth of its
        // time, and the 16-bit S cost accuracy: about 1e-4 of the result, enough to round 2 % of the outputs the other
        // way.)
        const uint32_t sbw[4] = {sb4.x, sb4.y, sb4.z, sb4.w};
        float xs[MT][2];
#pragma unroll
        for (int jj = 0; jj < MT; jj++) {
            const float2 sv = *reinterpret_cast<const float2*>(stage + sum_off[jj]);
            xs[jj][0] = sv.x;
            xs[jj][1] = sv.y;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[st]);   // everything of this stage is in registers now
#pragma unroll
        for (int s = 0; s < 2; s++) {
            const float s0 = bf_lo(sbw[2 * s]), s1 = bf_lo(sbw[2 * s + 1]);
            const float c0 = fmaf(-128.f, s0, bf_hi(sbw[2 * s])), c1 = fmaf(-128.f, s1, bf_hi(sbw[2 * s + 1]));
#pragma unroll
            for (int jj = 0; jj < MT; jj++) {
                acc[s][jj][0] = fmaf(c0, xs[jj][0], fmaf(s0, d[s][jj][0], acc[s][jj][0]));
                acc[s][jj][1] = fmaf(c0, xs[jj][1], fmaf(s0, d[s][jj][1], acc[s][jj][1]));
                acc[s][jj][2] = fmaf(c1, xs[jj][0], fmaf(s1, d[s][jj][2], acc[s][jj][2]));
                acc[s][jj][3] = fmaf(c1, xs[jj][1], fmaf(s1, d[s][jj][3], acc[s][jj][3]));
            }
        }
        }
        if (++kg == p.G) {
            flush(sb, seg_kg0, p.G);
            kg = 0; seg_kg0 = 0; sb++;
        }
    }
#if defined(VK_TRACE) && VK_TRACE == 2
    const long long tc_loop = clock64() - tc_t0;
#endif
    if (ok && kg != seg_kg0) flush(sb, seg_kg0, kg);
#if defined(VK_TRACE) && VK_TRACE == 2
    if (threadIdx.x == 32) {
        g_vk_trace[(blockIdx.x & 4095) * 16 + 3] = tc_wait;                 // consumer warp 0: cycles waiting for data
        g_vk_trace[(blockIdx.x & 4095) * 16 + 4] = tc_loop;                 // consumer warp 0: cycles in the step loop
        g_vk_trace[(blockIdx.x & 4095) * 16 + 6] = clock64() - tc_t0;       // ... including the final flush
    }
#endif
    // (a timed-out wait leaves the output unwritten and the status word set; copies still in flight land in this
    // CTA's shared memory, which stays allocated until the last warp of the CTA has left, after its own bounded waits)
}

// ------------------------------------------------------------------------------------------------ x records
// x [M, ldx] row-major bf16 -> [G] records (see the file comment). One CTA of 128 threads per group: thread (m, c)
// moves the 16-byte piece c of row m and the eight lanes of a row add up its 64 values (each lane its 8 in order,
// then an xor tree over the lanes).
// (grid.y = records per group: record r of a group holds rows 16 r .. 16 r + 15, the records of a group lie together)
__global__ void __launch_bounds__(128) w4_xrec_kernel(const __nv_bfloat16* __restrict__ x, int ldx, int M, uint8_t* __restrict__ xrec) {
    pdl_launch_dependents();
    pdl_wait();
    const int kg = blockIdx.x, rec = blockIdx.y, ml = threadIdx.x >> 3, c = threadIdx.x & 7;
    const int m = rec * 16 + ml;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (m < M) v = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + kg * 64 + c * 8);
    float f[8] = {bf_lo(v.x), bf_hi(v.x), bf_lo(v.y), bf_hi(v.y), bf_lo(v.z), bf_hi(v.z), bf_lo(v.w), bf_hi(v.w)};
    xrec_store_row_piece(xrec + ((size_t)kg * gridDim.y + rec) * kXRecBytes, ml, c, f);
}

// ------------------------------------------------------------------------------------------------ repack / dequant
// reference layout -> packed chunks. One thread per packed u32 (codes) or per scale word.
__global__ void w4_repack_kernel(const uint32_t* __restrict__ w, const __nv_bfloat16* __restrict__ sc,
                                 const __nv_bfloat16* __restrict__ bi, int N, int K, int group, uint8_t* __restrict__ out,
                                 int NSB, int G) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)NSB * G * kBlocksPerSB * 288;  // u32 words per chunk
    if (idx >= total) return;
    const size_t chunk = idx / 288;
    const int wi = (int)(idx - chunk * 288);
    const int jb = (int)(chunk % kBlocksPerSB);
    const size_t step = chunk / kBlocksPerSB;
    const int sbk = (int)(step / G), kg = (int)(step - (size_t)sbk * G);
    const int nb = sbk * kBlocksPerSB + jb;
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
        const int jx = wi - 256;  // [g][4]
        const int g = jx >> 2, e = jx & 3;
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
    for (int jx = 0; jx < 4; jx++) {
        const __nv_bfloat16 u0 = __ushort_as_bfloat16((unsigned short)(0x4300u | ((word >> (8 * jx)) & 0xFu)));
        const __nv_bfloat16 u1 = __ushort_as_bfloat16((unsigned short)(0x4300u | ((word >> (8 * jx + 4)) & 0xFu)));
        const __nv_bfloat16 k128 = __ushort_as_bfloat16((unsigned short)0x4300u);
        const __nv_bfloat16 r0 = __hfma(__hsub(u0, k128), s, b);   // 128 + u - 128 is exact
        const __nv_bfloat16 r1 = __hfma(__hsub(u1, k128), s, b);
        o[jx] = (uint32_t)__bfloat16_as_ushort(r0) | ((uint32_t)__bfloat16_as_ushort(r1) << 16);
    }
    *reinterpret_cast<uint4*>(out + (size_t)n * K + (size_t)wi * 8) = make_uint4(o[0], o[1], o[2], o[3]);
}

// row-major bf16 W [N, K] -> 4096-byte chunks in fragment order. One thread per u32 (two consecutive columns).
__global__ void bf16_repack_kernel(const __nv_bfloat16* __restrict__ W, int N, int K, uint8_t* __restrict__ out, int NSB, int G) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)NSB * G * kBlocksPerSB * 1024;
    if (idx >= total) return;
    const size_t chunk = idx >> 10;
    const int wi = (int)(idx & 1023);
    const int jb = (int)(chunk % kBlocksPerSB);
    const size_t step = chunk / kBlocksPerSB;
    const int sbk = (int)(step / G), kg = (int)(step - (size_t)sbk * G);
    const int nb = sbk * kBlocksPerSB + jb;
    const int i = wi & 3, lane = (wi >> 2) & 31, q = (wi >> 7) & 3, s = wi >> 9;
    const int g = lane >> 2, t = lane & 3;
    const int r = nb * 32 + s * 16 + g + (i & 1) * 8;
    const int c = kg * 64 + q * 16 + 2 * t + (i >> 1) * 8;
    uint32_t v = 0;
    if (r < N) v = *reinterpret_cast<const uint32_t*>(W + (size_t)r * K + c);
    reinterpret_cast<uint32_t*>(out)[idx] = v;
}

// 0 (default): up to 16 activation rows run on w4_gemm_kernel<MT, 0> (mma.sync); 2 / 3: on w4_t5_kernel (tcgen05 per
// group, w4_t5.cu) with that many steps between a warp's expansion and accumulation of a step; 4: on w4_tacc_kernel
// (dequantised weights, accumulation in tensor memory, w4_tacc.cu). Both tcgen05 forms are measured slower.
int g_w4_t5 = 0;
struct W4Params;
cudaError_t w4_t5_launch(const W4Params& p, cudaStream_t stream);
cudaError_t w4_tacc_launch(const W4Params& p, cudaStream_t stream);
cudaError_t w4_tacc_launch128(const W4Params& p, cudaStream_t stream);

int g_force_ctas = 0;
int g_prefetch_mb = 0;    // L2 prefetch budget of one GEMM launch in MB; off by default: measured slower (it competes with demand loads)

// steps per CTA beyond the smem ring that fit the prefetch budget
static int w4_prefetch_steps(int ctas, size_t stage_bytes, int stages) {
    const long long per_cta = (long long)g_prefetch_mb * 1000000ll / ((long long)ctas * (long long)stage_bytes) - stages;
    return per_cta < 0 ? 0 : (per_cta > 4096 ? 4096 : (int)per_cta);
}

struct W4Plan {
    int P, maxc, NSB, G, S;
    long long T;
};

W4Plan w4_plan(int N, int K, int ctas_per_sm = Fmt<0>::kCtasPerSM) {
    W4Plan pl;
    pl.NSB = (N + kSBRows - 1) / kSBRows;
    pl.G = K / 64;
    pl.T = (long long)pl.NSB * pl.G;
    int P = ctas_per_sm * 148;             // every CTA resident at once
    pl.S = 0;
    // Few superblocks (N small against the SM count): give every superblock the same number S of CTAs, each an
    // equal slice of K, so that the S partial sums of a superblock are ready together and its CTAs share the final
    // addition. Otherwise: equal contiguous ranges of the (superblock, group) sequence.
    if (g_force_ctas == 0 && pl.NSB * 4 <= P && pl.NSB <= 2048) {
        int S = P / pl.NSB;
        if (S > pl.G) S = pl.G;
        if (S >= 2) {
            pl.S = S;
            pl.P = pl.NSB * S;
            pl.maxc = S;
            return pl;
        }
    }
    if (g_force_ctas > 0) P = g_force_ctas;
    if ((long long)P > pl.T) P = (int)pl.T;
    pl.P = P;
    // the largest number of ranges that meet one superblock
    int maxc = 1;
    for (int sb = 0; sb < pl.NSB; sb++) {
        const long long s0 = (long long)sb * pl.G;
        const int c0 = (int)(((s0 + 1) * P - 1) / pl.T), c1 = (int)(((s0 + pl.G) * P - 1) / pl.T);
        maxc = c1 - c0 + 1 > maxc ? c1 - c0 + 1 : maxc;
    }
    pl.maxc = maxc;
    return pl;
}

// counters | x records [G][nrec] | partial sums [NSB][maxc][256][ps] fp32
size_t w4_ws_bytes(const W4Plan& pl, int nrec = 1, int ps = 16) {
    return kCounterBytes + (size_t)pl.G * nrec * kXRecBytes + (size_t)pl.NSB * pl.maxc * kSBRows * ps * 4;
}

template <int MT>
static cudaError_t w4_launch_pass(const void* packed, const __nv_bfloat16* x, int ldx, __nv_bfloat16* y, int ldy, int m, int N,
                                  int K, uint8_t* ws, cudaStream_t stream) {
    constexpr int NR = n_records<MT>(), PS = MT * 8 < 16 ? 16 : MT * 8;
    const bool t5 = MT <= 2 && g_w4_t5 != 0;
    const W4Plan pl = w4_plan(N, K, t5 ? 1 : ctas_per_sm<0, MT>());
    static PerDeviceOnce once;
    cudaError_t e = once.run([] {
        cudaError_t r = cudaFuncSetAttribute(w4_gemm_kernel<MT, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<0, MT>());
        if (r != cudaSuccess) return r;
        return cudaFuncSetAttribute(w4_gemm_kernel<MT, 0>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    });
    if (e != cudaSuccess) return e;
    W4Params p;
    p.wp = (const uint8_t*)packed;
    p.xrec = ws + kCounterBytes;
    p.y = y;
    p.counters = (int*)ws;
    p.part = (float*)(ws + kCounterBytes + (size_t)pl.G * NR * kXRecBytes);
    p.T = pl.T; p.M = m; p.N = N; p.NSB = pl.NSB; p.G = pl.G; p.P = pl.P; p.ldy = ldy; p.maxc = pl.maxc; p.S = pl.S;
    p.pf = w4_prefetch_steps(pl.P, (size_t)wstage_bytes<0>(), Fmt<0>::kStages);
    (void)PS;
    e = vk_launch(w4_xrec_kernel, dim3(pl.G, NR), dim3(128), 0, stream, x, ldx, m, ws + kCounterBytes);
    if (e != cudaSuccess) return e;
    if (t5) return g_w4_t5 == 4 ? w4_tacc_launch(p, stream) : w4_t5_launch(p, stream);
    return vk_launch(w4_gemm_kernel<MT, 0>, dim3(pl.P), dim3(kThreads), smem_bytes<0, MT>(), stream, p);
}

}  // namespace

extern "C" {

size_t vk_w4_packed_bytes(int N, int K) { return (size_t)((N + kSBRows - 1) / kSBRows) * (K / 64) * wstage_bytes<0>(); }

int vk_w4_repack(const void* w, const void* scales, const void* biases, int N, int K, int group, void* packed,
                 cudaStream_t stream) {
    if (N <= 0 || K <= 0 || K % 64 != 0 || (group != 64 && group != 128) || K % group != 0) return VK_EINVAL;
    const int NSB = (N + kSBRows - 1) / kSBRows, G = K / 64;
    const size_t total = (size_t)NSB * G * kBlocksPerSB * 288;
    w4_repack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
        (const uint32_t*)w, (const __nv_bfloat16*)scales, (const __nv_bfloat16*)biases, N, K, group, (uint8_t*)packed, NSB, G);
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

void vk_w4_force_plan(int ctas, int prefetch_mb) {
    g_force_ctas = ctas;
    g_prefetch_mb = prefetch_mb < 0 ? 0 : prefetch_mb;
}

void vk_w4_select(int form) { g_w4_t5 = form < 0 ? 0 : form; }

size_t vk_w4_workspace_bytes(int M, int N, int K) {
    if (N <= 0 || K <= 0 || K % 64 != 0) return 0;
    size_t need = w4_ws_bytes(w4_plan(N, K));
    const size_t one = w4_ws_bytes(w4_plan(N, K, 1));   // (the tcgen05 kernel runs one CTA per SM)
    need = one > need ? one : need;
    if (M > 16) {   // passes of 32 / 64 rows: one CTA per SM, wider records and partial sums
        const size_t wide = w4_ws_bytes(w4_plan(N, K, 1), M > 32 ? 4 : 2, M > 32 ? 64 : 32);
        need = wide > need ? wide : need;
    }
    return need;
}

// y = x . dequant(W)^T for activations already laid out as x records (K / 64 records of 2176 bytes, rows >= M zero):
// what the fused producers of this library write. M <= 16.
int vk_w4_gemm_xrec(const void* packed, const void* xrec, void* y, int ldy, int M, int N, int K, void* workspace,
                    size_t workspace_bytes, cudaStream_t stream) {
    if (M <= 0 || M > 16 || N <= 0 || K <= 0 || K % 64 != 0 || ldy < N) return VK_EINVAL;
    if (((uintptr_t)xrec & 15) || ((uintptr_t)packed & 15) || workspace == nullptr || ((uintptr_t)workspace & 15)) return VK_EINVAL;
    const bool t5 = g_w4_t5 != 0;
    const W4Plan pl = w4_plan(N, K, t5 ? 1 : Fmt<0>::kCtasPerSM);
    if (pl.NSB > (int)(kCounterBytes / 8)) return VK_EINVAL;
    if (workspace_bytes < w4_ws_bytes(pl)) return VK_ENOSPC;
    static PerDeviceOnce once;
    if (!t5) {
        VK_CUDA(once.run([] {
            cudaError_t r = cudaFuncSetAttribute(w4_gemm_kernel<1, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<0>());
            if (r == cudaSuccess) r = cudaFuncSetAttribute(w4_gemm_kernel<1, 0>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            if (r == cudaSuccess) r = cudaFuncSetAttribute(w4_gemm_kernel<2, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<0>());
            if (r == cudaSuccess) r = cudaFuncSetAttribute(w4_gemm_kernel<2, 0>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            return r;
        }));
    }
    uint8_t* ws = (uint8_t*)workspace;
    W4Params p;
    p.wp = (const uint8_t*)packed;
    p.xrec = (const uint8_t*)xrec;
    p.y = (__nv_bfloat16*)y;
    p.counters = (int*)ws;
    p.part = (float*)(ws + kCounterBytes + (size_t)pl.G * kXRecBytes);
    p.T = pl.T; p.M = M; p.N = N; p.NSB = pl.NSB; p.G = pl.G; p.P = pl.P; p.ldy = ldy; p.maxc = pl.maxc; p.S = pl.S;
    p.pf = w4_prefetch_steps(pl.P, (size_t)wstage_bytes<0>(), Fmt<0>::kStages);
    if (t5) return (int)(g_w4_t5 == 4 ? w4_tacc_launch(p, stream) : w4_t5_launch(p, stream));
    cudaError_t e = M <= 8 ? vk_launch(w4_gemm_kernel<1, 0>, dim3(pl.P), dim3(kThreads), smem_bytes<0>(), stream, p)
                           : vk_launch(w4_gemm_kernel<2, 0>, dim3(pl.P), dim3(kThreads), smem_bytes<0>(), stream, p);
    return (int)e;
}

// Row-major x. Up to 16 rows: one pass (two CTAs per SM). More rows (verify windows, prefill chunks): passes of 64,
// then 32, then up to 16 rows, each streaming the weights once; the wide passes keep 8 / 4 row tiles per warp and run
// one CTA per SM.
int vk_w4_gemm(const void* packed, const void* x, int ldx, void* y, int ldy, int M, int N, int K, void* workspace,
               size_t workspace_bytes, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0 || K % 64 != 0 || ldx % 8 != 0 || ldx < K || ldy < N) return VK_EINVAL;
    if (((uintptr_t)x & 15) || ((uintptr_t)packed & 15) || workspace == nullptr || ((uintptr_t)workspace & 15)) return VK_EINVAL;
    const W4Plan pl = w4_plan(N, K);
    if (pl.NSB > (int)(kCounterBytes / 4)) return VK_EINVAL;
    if (workspace_bytes < vk_w4_workspace_bytes(M, N, K)) return VK_ENOSPC;
    uint8_t* ws = (uint8_t*)workspace;
    for (int m0 = 0; m0 < M;) {
        const int left = M - m0;
        const __nv_bfloat16* xp = (const __nv_bfloat16*)x + (size_t)m0 * ldx;
        __nv_bfloat16* yp = (__nv_bfloat16*)y + (size_t)m0 * ldy;
        cudaError_t e;
        int m;
        if (left > 32) { m = left < 64 ? left : 64; e = w4_launch_pass<8>(packed, xp, ldx, yp, ldy, m, N, K, ws, stream); }
        else if (left > 16) { m = left; e = w4_launch_pass<4>(packed, xp, ldx, yp, ldy, m, N, K, ws, stream); }
        else if (left > 8) { m = left; e = w4_launch_pass<2>(packed, xp, ldx, yp, ldy, m, N, K, ws, stream); }
        else { m = left; e = w4_launch_pass<1>(packed, xp, ldx, yp, ldy, m, N, K, ws, stream); }
        if (e != cudaSuccess) return (int)e;
        m0 += m;
    }
    return VK_OK;
}

// ---- the same streaming kernel over plain bf16 weights (lm_head and the other unquantised linears)
size_t vk_bf16_packed_bytes(int N, int K) { return (size_t)((N + kSBRows - 1) / kSBRows) * (K / 64) * wstage_bytes<1>(); }

int vk_bf16_repack(const void* W, int N, int K, void* packed, cudaStream_t stream) {
    if (N <= 0 || K <= 0 || K % 64 != 0) return VK_EINVAL;
    const int NSB = (N + kSBRows - 1) / kSBRows, G = K / 64;
    const size_t total = (size_t)NSB * G * kBlocksPerSB * 1024;
    bf16_repack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)W, N, K, (uint8_t*)packed, NSB, G);
    return (int)cudaGetLastError();
}

size_t vk_bf16_workspace_bytes(int M, int N, int K) {
    (void)M;
    if (N <= 0 || K <= 0 || K % 64 != 0) return 0;
    return w4_ws_bytes(w4_plan(N, K, Fmt<1>::kCtasPerSM));
}

int vk_bf16_gemm_packed(const void* packed, const void* x, int ldx, void* y, int ldy, int M, int N, int K, void* workspace,
                        size_t workspace_bytes, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0 || K % 64 != 0 || ldx % 8 != 0 || ldx < K || ldy < N) return VK_EINVAL;
    if (((uintptr_t)x & 15) || ((uintptr_t)packed & 15) || workspace == nullptr || ((uintptr_t)workspace & 15)) return VK_EINVAL;
    const W4Plan pl = w4_plan(N, K, Fmt<1>::kCtasPerSM);
    if (pl.NSB > (int)(kCounterBytes / 4)) return VK_EINVAL;
    if (workspace_bytes < w4_ws_bytes(pl)) return VK_ENOSPC;
    static PerDeviceOnce once;
    VK_CUDA(once.run([] {
        cudaError_t r = cudaFuncSetAttribute(w4_gemm_kernel<1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<1>());
        if (r == cudaSuccess) r = cudaFuncSetAttribute(w4_gemm_kernel<1, 1>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (r == cudaSuccess) r = cudaFuncSetAttribute(w4_gemm_kernel<2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<1>());
        if (r == cudaSuccess) r = cudaFuncSetAttribute(w4_gemm_kernel<2, 1>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        return r;
    }));
    uint8_t* ws = (uint8_t*)workspace;
    for (int m0 = 0; m0 < M; m0 += 16) {
        const int m = M - m0 < 16 ? M - m0 : 16;
        W4Params p;
        p.wp = (const uint8_t*)packed;
        p.xrec = ws + kCounterBytes;
        p.y = (__nv_bfloat16*)y + (size_t)m0 * ldy;
        p.counters = (int*)ws;
        p.part = (float*)(ws + kCounterBytes + (size_t)pl.G * kXRecBytes);
        p.T = pl.T; p.M = m; p.N = N; p.NSB = pl.NSB; p.G = pl.G; p.P = pl.P; p.ldy = ldy; p.maxc = pl.maxc; p.S = pl.S;
        p.pf = w4_prefetch_steps(pl.P, (size_t)wstage_bytes<1>(), Fmt<1>::kStages);
        VK_CUDA(vk_launch(w4_xrec_kernel, dim3(pl.G), dim3(128), 0, stream, (const __nv_bfloat16*)x + (size_t)m0 * ldx, ldx, m,
                          ws + kCounterBytes));
        cudaError_t e = m <= 8 ? vk_launch(w4_gemm_kernel<1, 1>, dim3(pl.P), dim3(kThreads), smem_bytes<1>(), stream, p)
                               : vk_launch(w4_gemm_kernel<2, 1>, dim3(pl.P), dim3(kThreads), smem_bytes<1>(), stream, p);
        if (e != cudaSuccess) return (int)e;
    }
    return VK_OK;
}

}  // extern "C"
