// INT4 affine weight GEMM for many activation rows (verify windows of B x T rows, prefill chunks) on the 5th-generation
// tensor cores: y[M, N] = x[M, K] . dequant(w)[N, K]^T with tcgen05.mma, the accumulator in tensor memory.
//
// Replaces mx.quantized_matmul at M = B * T or a prefill chunk (batch_spec.verify_forward, batch_spec.py:107-158;
// session.prefill_iter, session.py:351-387): there the product is compute-bound, so unlike the small-M kernel
// (w4_gemm.cu), which multiplies raw codes and applies scale and bias to the group's fp32 product, this one
// dequantises a weight tile to bf16 once, bf16(s * u + b) rounded once (mx.dequantize's value, vk_w4_dequant), and feeds
// it to the tensor cores; the activations are used as they are. It reads the same packed weights (vk_w4_repack).
//
// One CTA = one 256-row superblock of the weight (the D tile's N) x 128 activation rows (the D tile's M) x all of K:
//   warp 0      one lane: 1-D TMA bulk copies per 64-column group: the packed 9216-byte weight step and the 16 KB
//               activation tile (pre-arranged by w4_xtile_kernel) into a 3-stage ring
//   warp 1      one lane: waits for a stage's activations and dequantised weights, issues 4 tcgen05.mma (M 128, N 256,
//               K 16, A and B from shared memory, K-major, no swizzle), commits them to the stage's "free" barrier
//   warps 2..9  dequantisers: unpack the codes of the stage (the mma.sync fragment order of the packed layout),
//               bf16(s * u + b) with one fused rounding, store into the canonical K-major layout, fence to the async
//               proxy, arrive on the stage's "weights ready" barrier
//   warps 4..7  afterwards: tcgen05.ld of their 32 accumulator lanes (= activation rows), bf16, 16-byte stores
// Shared-memory operand layout (both operands, "K-major interleaved", 16-byte units): [k / 8][row][8 elements]: a core
// matrix is 8 rows x 16 bytes, contiguous; leading-dimension (K) offset = rows * 16 bytes, stride (row group) offset
// = 128 bytes.
// Every wait is bounded: a wait that runs out sets the status word, the kernel skips ahead, frees its tensor memory
// and returns.
#include "common.cuh"

namespace {

constexpr int kTileM = 128;                    // activation rows per CTA = accumulator lanes
constexpr int kPackedStep = 9216;              // bytes of one (superblock, group) of packed weights
constexpr int kXTileBytes = kTileM * 64 * 2;   // 16 KB: [8][128][8] bf16
constexpr int kDqWarps = 8;                    // dequantiser warps (16 measured the same: the kernel is not bound by them)
constexpr int kTileThreads = 64 + 32 * kDqWarps;
// Weight rows per CTA = accumulator columns: TN = 256 (a whole superblock) for weights with many rows; TN = 64 (a
// quarter: two of the superblock's eight 32-row chunks) for weights whose 256-row tiles would not fill the GPU.
// ML = tiles of 128 activation rows per CTA (1 or 2): with two, every dequantised weight tile feeds two accumulators,
// which halves the dequantisation work per multiply-add (the limit of this kernel).
template <int TN, int ML> struct TileCfg {
    static constexpr int kPacked = TN / 32 * 1152;          // bytes of the CTA's chunks inside a packed step
    static constexpr int kWd = TN * 64 * 2;                  // dequantised tile [8][TN][8] bf16
    static constexpr int kStage = kPacked + ML * kXTileBytes + kWd;
    static constexpr int kStages = (220 * 1024 / kStage) < 6 ? (220 * 1024 / kStage) : 6;
    static constexpr int kSplit = kDqWarps / (TN / 32);      // dequantiser warps per 32-row chunk: all of them work
    static constexpr int kBarBytes = (3 * kStages + 1) * 8;  // full / wready / freeb per stage + accdone
    static constexpr size_t kSmem = (size_t)kStages * kStage + ((kBarBytes + 127) / 128) * 128;
    static_assert(kSmem <= 227 * 1024, "stages do not fit the CTA's shared memory");
    static constexpr uint32_t kCols = TN * ML;               // tensor-memory columns (a power of two >= 32)
};

struct TileParams {
    const uint8_t* wp;        // packed weights [NSB][G][9216]
    const uint8_t* xt;        // activation tiles [MT][G][16 KB]
    __nv_bfloat16* y;         // [M, ldy]
    int M, N, G, ldy;
};

// x [M, ldx] row-major -> tiles [M / 128][G][k / 8 (8)][row (128)][8 bf16]; rows beyond M are zero
__global__ void __launch_bounds__(128) w4_xtile_kernel(const __nv_bfloat16* __restrict__ x, int ldx, int M, int G,
                                                       uint8_t* __restrict__ xt) {
    pdl_launch_dependents();
    pdl_wait();
    const int kg = blockIdx.x, mt = blockIdx.y, r = threadIdx.x;
    const int m = mt * kTileM + r;
    uint8_t* dst = xt + ((size_t)mt * G + kg) * kXTileBytes;
#pragma unroll
    for (int c = 0; c < 8; c++) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (m < M) v = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + kg * 64 + c * 8);
        *reinterpret_cast<uint4*>(dst + ((size_t)c * kTileM + r) * 16) = v;
    }
}

int g_tile_force_tn = 0, g_tile_force_ml = 0;

__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    // start address, leading-dimension and stride byte offsets in 16-byte units; version 1 (sm_100); no swizzle
    return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46);
}

template <int TN, int ML>
__global__ void __launch_bounds__(kTileThreads, 1) w4_tile_kernel(const TileParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    using Cfg = TileCfg<TN, ML>;
    constexpr int kTileN = TN;
    constexpr int kTStages = Cfg::kStages;
    constexpr int kTStageBytes = Cfg::kStage;
    constexpr int kPackedBytes = Cfg::kPacked;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kTStages * kTStageBytes);
    uint64_t* full = bars;                   // [stage] packed weights + activation tile have landed (TMA bytes)
    uint64_t* wready = bars + kTStages;      // [stage] dequantised weights are in place (every dequantiser thread arrives)
    uint64_t* freeb = bars + 2 * kTStages;   // [stage] the stage's MMAs have finished reading it
    uint64_t* accdone = bars + 3 * kTStages; // the whole accumulation has finished
    __shared__ uint32_t s_tmem;
    __shared__ int s_fail;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int kPerSB = 256 / TN;                     // CTAs per superblock
    const int sb = blockIdx.x / kPerSB, part = blockIdx.x % kPerSB, mt = blockIdx.y * ML;
    const int n_base = sb * 256 + part * TN;             // first weight row of this CTA
    const int G = p.G;
    const int nm = (ML == 2 && (mt + 1) * kTileM < p.M) ? 2 : 1;   // tiles of activation rows this CTA really has

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTStages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&wready[s], 32 * kDqWarps);
            mbar_init(&freeb[s], 1);
        }
        mbar_init(accdone, 1);
        mbar_fence_init();
        s_fail = 0;
    }
    if (warp == 1) {   // one warp allocates the accumulator: 256 columns of tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(Cfg::kCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            const uint8_t* wsrc = p.wp + (size_t)sb * G * kPackedStep + (size_t)part * kPackedBytes;
            const uint8_t* xsrc = p.xt + (size_t)mt * G * kXTileBytes;
            pdl_wait();
            pdl_launch_dependents();
            int st = 0;
            uint32_t par = 0;
            for (int i = 0; i < G; i++) {
                if (i >= kTStages && !mbar_wait(&freeb[st], par)) { s_fail = 1; break; }
                fence_proxy_async_smem();   // (the expansion warps read the packed codes with ld.shared)
                uint8_t* dst = smem + (size_t)st * kTStageBytes;
                mbar_expect_tx(&full[st], kPackedBytes + nm * kXTileBytes);
                tma_bulk_g2s(dst, wsrc + (size_t)i * kPackedStep, kPackedBytes, &full[st]);
                tma_bulk_g2s(dst + kPackedBytes, xsrc + (size_t)i * kXTileBytes, kXTileBytes, &full[st]);
                if (nm == 2)
                    tma_bulk_g2s(dst + kPackedBytes + kXTileBytes, xsrc + ((size_t)G + i) * kXTileBytes, kXTileBytes, &full[st]);
                if (++st == kTStages) { st = 0; if (i >= kTStages) par ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0) {
            // instruction descriptor: D fp32, A and B bf16, both K-major, N = TN, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kTileN >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
            int st = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int i = 0; i < G && ok; i++) {
                if (!mbar_wait(&full[st], ph) || !mbar_wait(&wready[st], ph)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a0 = smem_u32(smem + (size_t)st * kTStageBytes + kPackedBytes);
                const uint32_t b0 = a0 + ML * kXTileBytes;
#pragma unroll
                for (int kk = 0; kk < 4; kk++) {   // K = 16 per instruction = two 16-byte units along K
                    const uint64_t db = umma_desc(b0 + kk * 2 * (kTileN * 16), kTileN * 16, 128);
                    const uint32_t accumulate = (i > 0 || kk > 0) ? 1u : 0u;
                    const uint32_t zero = 0u;   // (no output lane disabled)
#pragma unroll
                    for (int mi = 0; mi < ML; mi++) {   // accumulator mi: columns mi TN .. of tensor memory
                        if (mi < nm) {
                            const uint64_t da = umma_desc(a0 + mi * kXTileBytes + kk * 2 * (kTileM * 16), kTileM * 16, 128);
                            asm volatile(
                                "{\n\t"
                                ".reg .pred p;\n\t"
                                "setp.ne.b32 p, %4, 0;\n\t"
                                "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
                                "}\n" ::"r"(tmem + (uint32_t)(mi * TN)), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(zero)
                                : "memory");
                        }
                    }
                }
                // the stage may be refilled once these MMAs have read it (the commit also fences the issue order)
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&freeb[st]))
                             : "memory");
                if (++st == kTStages) { st = 0; ph ^= 1u; }
            }
            if (!ok) s_fail = 1;
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(accdone))
                         : "memory");
        }
    } else {
        // ---------------------------------------------------------------- dequantisers (warps 2 ..)
        // A chunk of 32 rows x 64 columns is 2 (s: 16 rows) x 4 (q: 16 columns) words per lane, shared by the kSplit
        // warps of the chunk: one warp takes all eight words, two take one s each, four (s, two q), eight (s, q).
        constexpr int kSplit = Cfg::kSplit;
        static_assert(kSplit == 1 || kSplit == 2 || kSplit == 4 || kSplit == 8, "dequantiser warps per chunk");
        constexpr int kQ = kSplit == 1 ? 4 : 8 / kSplit;          // words of one s per thread
        constexpr int kPerS = kSplit == 1 ? 1 : kSplit / 2;        // warps that share one s
        const int dw = (threadIdx.x - 64) >> 5;   // 0 .. kDqWarps - 1
        const int j = dw / kSplit;                // 32-row chunk of this CTA's rows
        const int sub = dw % kSplit;
        const int s_lo = kSplit == 1 ? 0 : sub / kPerS, s_hi = kSplit == 1 ? 2 : s_lo + 1;
        const int q_lo = (sub % kPerS) * kQ;
        const int g = lane >> 2, t = lane & 3;
        int st = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int i = 0; i < G; i++) {
            if (!mbar_wait(&full[st], ph)) { ok = false; break; }
            const uint8_t* stage = smem + (size_t)st * kTStageBytes;
            const uint8_t* ch = stage + j * 1152;
            uint8_t* wd = smem + (size_t)st * kTStageBytes + kPackedBytes + ML * kXTileBytes;
            const uint4 sb4 = *reinterpret_cast<const uint4*>(ch + 1024 + g * 16);   // (scale | bias << 16) of 4 rows
#pragma unroll
            for (int s = s_lo; s < s_hi; s++) {
                uint32_t wq[kQ];
                if constexpr (kQ == 4) {
                    const uint4 wv = *reinterpret_cast<const uint4*>(ch + s * 512 + lane * 16);
                    wq[0] = wv.x, wq[1] = wv.y, wq[2] = wv.z, wq[3] = wv.w;
                } else if constexpr (kQ == 2) {
                    const uint2 wv = *reinterpret_cast<const uint2*>(ch + s * 512 + lane * 16 + q_lo * 4);
                    wq[0] = wv.x, wq[1] = wv.y;
                } else {
                    wq[0] = *reinterpret_cast<const uint32_t*>(ch + s * 512 + lane * 16 + q_lo * 4);
                }
                // rows n0 = 32 j + 16 s + g and n0 + 8; their scale / bias as bf16 pairs
                __nv_bfloat162 sc2[2], bi2[2];
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const uint32_t wsb = s ? (h ? sb4.w : sb4.z) : (h ? sb4.y : sb4.x);
                    const uint32_t ss = (wsb & 0xFFFFu) | (wsb << 16), bb = (wsb >> 16) | (wsb & 0xFFFF0000u);
                    sc2[h] = *reinterpret_cast<const __nv_bfloat162*>(&ss);
                    bi2[h] = *reinterpret_cast<const __nv_bfloat162*>(&bb);
                }
                const uint32_t c128 = 0x43004300u;
                const __nv_bfloat162 k128 = *reinterpret_cast<const __nv_bfloat162*>(&c128);
#pragma unroll
                for (int qi = 0; qi < kQ; qi++) {
                    const int q = q_lo + qi;
                    // register i of the word: (row n0 + 8 (i & 1), columns 16 q + 8 (i >> 1) + 2 t, + 1) as 128 + code
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        const uint32_t au = ((wq[qi] >> (4 * r)) & 0x000F000Fu) | 0x43004300u;
                        const __nv_bfloat162 u2 = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&au), k128);   // exact
                        const __nv_bfloat162 v2 = __hfma2(u2, sc2[r & 1], bi2[r & 1]);                            // one rounding
                        const int n = 32 * j + 16 * s + g + 8 * (r & 1);
                        const int kcol = 16 * q + 8 * (r >> 1) + 2 * t;
                        *reinterpret_cast<__nv_bfloat162*>(wd + ((size_t)(kcol >> 3) * kTileN + n) * 16 + (kcol & 7) * 2) = v2;
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> visible to the MMA
            mbar_arrive(&wready[st]);
            if (++st == kTStages) { st = 0; ph ^= 1u; }
        }
        if (!ok) s_fail = 1;
        // ---------------------------------------------------------------- epilogue (warps 4..7: lanes 32 (warp % 4) ..)
        static_assert(kDqWarps >= 6, "warps 4..7 read the accumulator");
        if (warp >= 4 && warp < 8) {
            if (ok && mbar_wait(accdone, 0)) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int mi = 0; mi < nm; mi++)
                for (int c0 = 0; c0 < kTileN; c0 += 8) {
                    const int m = (mt + mi) * kTileM + (warp & 3) * 32 + lane;
                    const uint32_t taddr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(mi * TN);
                    uint32_t r[8];
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                                 : "r"(taddr + (uint32_t)c0));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    const int n = n_base + c0;
                    if (m < p.M && n < p.N) {
                        __nv_bfloat16* dst = p.y + (size_t)m * p.ldy + n;
                        if (n + 8 <= p.N && ((((size_t)m * p.ldy + n) & 7) == 0)) {
                            uint4 o;
                            o.x = pack_bf2(__uint_as_float(r[0]), __uint_as_float(r[1]));
                            o.y = pack_bf2(__uint_as_float(r[2]), __uint_as_float(r[3]));
                            o.z = pack_bf2(__uint_as_float(r[4]), __uint_as_float(r[5]));
                            o.w = pack_bf2(__uint_as_float(r[6]), __uint_as_float(r[7]));
                            *reinterpret_cast<uint4*>(dst) = o;
                        } else {
#pragma unroll
                            for (int e = 0; e < 8; e++)
                                if (n + e < p.N) dst[e] = f2bf(__uint_as_float(r[e]));
                        }
                    }
                }
            } else {
                s_fail = 1;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(Cfg::kCols) : "memory");
    }
    if (threadIdx.x == 0 && s_fail) vk_set_status(VK_ST_MBAR_TIMEOUT);
}

}  // namespace

extern "C" {

// Test and tuning hook: force the tile shape (weight rows per CTA 256 / 64, activation-row tiles per CTA 1 / 2); 0 = automatic.
int vk_w4_tile_force(int tn, int ml) {
    if ((tn != 0 && tn != 64 && tn != 256) || ml < 0 || ml > 2) return VK_EINVAL;
    g_tile_force_tn = tn;
    g_tile_force_ml = ml;
    return VK_OK;
}

// Bytes of scratch vk_w4_gemm_tile needs for the re-arranged activations.
size_t vk_w4_tile_workspace_bytes(int M, int K) {
    if (M <= 0 || K <= 0 || K % 64 != 0) return 0;
    return (size_t)((M + kTileM - 1) / kTileM) * (K / 64) * kXTileBytes;
}

// Up to 128 rows run on the split-K kernel of w4_tacc.cu (every SM takes an equal range of the weight's steps, instead
// of whole superblocks in waves) when the workspace also holds its arrival counters and partial sums: this many bytes.
// With less (but at least vk_w4_tile_workspace_bytes) the call falls back to whole superblocks per CTA.
size_t vk_w4_tile_workspace_bytes_n(int M, int N, int K) {
    const size_t tiles = vk_w4_tile_workspace_bytes(M, K);
    if (tiles == 0 || N <= 0 || M > kTileM) return tiles;
    const W4Plan pl = w4_plan(N, K, 1);
    return kCounterBytes + tiles + (size_t)pl.NSB * pl.maxc * kSBRows * kTileM * sizeof(float);
}

static int g_tile_split = 1;   // 0: never the split-K kernel (test and measuring aid)
void vk_w4_tile_split(int on) { g_tile_split = on != 0; }

// y[M, N] = bf16(x[M, K] . dequant(W)^T) on tcgen05 tensor cores; `packed` as for vk_w4_gemm. Any M (tiles of 128 rows).
int vk_w4_gemm_tile(const void* packed, const void* x, int ldx, void* y, int ldy, int M, int N, int K, void* workspace,
                    size_t workspace_bytes, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0 || K % 64 != 0 || ldx % 8 != 0 || ldx < K || ldy < N) return VK_EINVAL;
    if (((uintptr_t)x & 15) || ((uintptr_t)packed & 15) || workspace == nullptr || ((uintptr_t)workspace & 15)) return VK_EINVAL;
    if (workspace_bytes < vk_w4_tile_workspace_bytes(M, K)) return VK_ENOSPC;
    static PerDeviceOnce once;
    VK_CUDA(once.run([] {
        cudaError_t r = cudaFuncSetAttribute(w4_tile_kernel<256, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TileCfg<256, 1>::kSmem);
        if (r == cudaSuccess) r = cudaFuncSetAttribute(w4_tile_kernel<256, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TileCfg<256, 2>::kSmem);
        if (r == cudaSuccess) r = cudaFuncSetAttribute(w4_tile_kernel<64, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TileCfg<64, 1>::kSmem);
        if (r == cudaSuccess) r = cudaFuncSetAttribute(w4_tile_kernel<64, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TileCfg<64, 2>::kSmem);
        return r;
    }));
    const int G = K / 64, MTn = (M + kTileM - 1) / kTileM, NSB = (N + 255) / 256;
    // (the split-K kernel pays for weights with few 256-row blocks, where whole blocks per CTA leave most SMs idle: its
    // partial sums are 128 KB per block and range, which costs more than it saves once every SM has a block of its own)
    const W4Plan pl = w4_plan(N, K, 1);
    if (MTn == 1 && g_tile_split && pl.S > 0 && g_tile_force_tn == 0 && g_tile_force_ml == 0 && NSB <= (int)(kCounterBytes / 8) &&
        workspace_bytes >= vk_w4_tile_workspace_bytes_n(M, N, K)) {
        uint8_t* ws = (uint8_t*)workspace;
        uint8_t* tiles = ws + kCounterBytes;
        VK_CUDA(vk_launch(w4_xtile_kernel, dim3(G, 1), dim3(128), 0, stream, (const __nv_bfloat16*)x, ldx, M, G, tiles));
        W4Params q;
        q.wp = (const uint8_t*)packed;
        q.xrec = tiles;
        q.y = (__nv_bfloat16*)y;
        q.counters = (int*)ws;     // (zero between launches: the kernels leave them so; the caller's buffer starts zeroed)
        q.part = (float*)(tiles + (size_t)G * kXTileBytes);
        q.T = pl.T; q.M = M; q.N = N; q.NSB = pl.NSB; q.G = pl.G; q.P = pl.P; q.ldy = ldy; q.maxc = pl.maxc; q.S = pl.S;
        q.pf = 0;
        return (int)w4_tacc_launch128(q, stream);
    }
    // (a workspace with room for it keeps its first 16 KB, the split-K form's arrival counters, untouched)
    uint8_t* xtiles = (uint8_t*)workspace;
    if (workspace_bytes >= kCounterBytes + vk_w4_tile_workspace_bytes(M, K)) xtiles += kCounterBytes;
    VK_CUDA(vk_launch(w4_xtile_kernel, dim3(G, MTn), dim3(128), 0, stream, (const __nv_bfloat16*)x, ldx, M, G, xtiles));
    TileParams p = {(const uint8_t*)packed, (const uint8_t*)xtiles, (__nv_bfloat16*)y, M, N, G, ldy};
    // Two tiles of activation rows per CTA when there are two; whole superblocks per CTA when that still gives at
    // least one CTA per two SMs, quarters of a superblock otherwise.
    const int ml = g_tile_force_ml ? g_tile_force_ml : (MTn >= 2 ? 2 : 1);
    const int gy = (MTn + ml - 1) / ml;
    const int tn = g_tile_force_tn ? g_tile_force_tn : (NSB * gy >= 74 ? 256 : 64);
    if (tn == 256 && ml == 2)
        return (int)vk_launch(w4_tile_kernel<256, 2>, dim3(NSB, gy), dim3(kTileThreads), TileCfg<256, 2>::kSmem, stream, p);
    if (tn == 256)
        return (int)vk_launch(w4_tile_kernel<256, 1>, dim3(NSB, gy), dim3(kTileThreads), TileCfg<256, 1>::kSmem, stream, p);
    if (ml == 2)
        return (int)vk_launch(w4_tile_kernel<64, 2>, dim3(NSB * 4, gy), dim3(kTileThreads), TileCfg<64, 2>::kSmem, stream, p);
    return (int)vk_launch(w4_tile_kernel<64, 1>, dim3(NSB * 4, gy), dim3(kTileThreads), TileCfg<64, 1>::kSmem, stream, p);
}

}  // extern "C"
