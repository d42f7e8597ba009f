// Shared device helpers for the sm_100a kernels: bf16 bit handling, bounded mbarrier waits, 1-D TMA bulk copies,
// programmatic dependent launch (PDL) and the launch wrapper every kernel in this library goes through.
#pragma once
#include <atomic>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define VK_OK 0
#define VK_EINVAL (-1)
#define VK_ENOSPC (-2)
#define VK_ETOOBIG (-3)  // the problem exceeds a fixed capacity of the entry point

// Device-side status word: 0 = fine; otherwise the code of the first kernel that gave up on a bounded wait or met
// an out-of-range index. Read (and cleared) by vk_status_read at the caller's sync point.
__device__ int g_vk_status = 0;  // (the library is one translation unit: volundr_b200.cu)
enum : int {
    VK_ST_MBAR_TIMEOUT = 1,   // a TMA bulk copy did not complete within the spin limit
    VK_ST_BAD_INDEX = 2,      // page / block index outside its pool
    VK_ST_POOL_EMPTY = 3,     // the page allocator ran out of free pages
    VK_ST_FLAG_TIMEOUT = 4,   // a split-K / peer flag wait ran out
};

__device__ __forceinline__ void vk_set_status(int code) { atomicCAS(&g_vk_status, 0, code); }

// Phase time stamps inside one kernel, for tuning builds only (-DVK_TRACE=<kernel id>): thread 0 of every CTA stores
// the SM's cycle counter at the marked points; vk_trace_read copies the table out. Compiled out otherwise.
#ifdef VK_TRACE
__device__ long long g_vk_trace[4096 * 16];
#define VK_TS(kernel_id, i)                                                                                      \
    do {                                                                                                         \
        if (VK_TRACE == (kernel_id) && threadIdx.x == 0)                                                         \
            g_vk_trace[(((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) & 4095) * 16 + (i)] = clock64(); \
    } while (0)
#else
#define VK_TS(kernel_id, i) do { } while (0)
#endif

// ---------------------------------------------------------------- bf16 <-> fp32 on raw bits
__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }
__device__ __forceinline__ float bf2f(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ __nv_bfloat16 f2bf(float x) { return __float2bfloat16_rn(x); }
// fp32 -> the fp32 value of its bf16 rounding (round to nearest even)
__device__ __forceinline__ float bfr(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ uint32_t pack_bf2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// ---------------------------------------------------------------- warp / block reductions (fixed order)
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Sum over a block of NW warps; `red` holds NW floats of shared memory. Every thread gets the total. The order of
// the additions is fixed (xor tree inside a warp, then warps 0..NW-1), so results do not depend on scheduling.
template <int NW>
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < NW; i++) t += red[i];
    return t;
}

// ---------------------------------------------------------------- mbarrier + TMA bulk (1-D) copies
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Pull `bytes` (a multiple of 16, 16-byte aligned) into L2 without waiting for them: used for weights that a kernel
// will read after its dependency wait, issued before that wait (weights depend on no earlier kernel).
__device__ __forceinline__ void l2_prefetch_bulk(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// ---------------------------------------------------------------- cp.async (16-byte copies global -> shared)
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait0() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t phase) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(phase)
        : "memory");
    return ok != 0;
}
// Non-blocking look at the barrier: true when phase `phase` has completed. (try_wait may suspend the thread for a while
// even when the phase is already complete; a plain test returns at shared-memory latency.)
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t phase) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(phase)
        : "memory");
    return ok != 0;
}
// Wait for phase `phase` of `bar` with an iteration limit. Returns false (and records VK_ST_MBAR_TIMEOUT) when the
// limit runs out, so a copy that never lands ends the kernel instead of hanging the GPU.
#define VK_MBAR_SPIN_LIMIT (1u << 20)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t phase) {
#ifndef VK_NO_TEST_WAIT
    if (mbar_test_wait(bar, phase)) return true;
#endif
    for (uint32_t i = 0; i < VK_MBAR_SPIN_LIMIT; i++) {
        if (mbar_try_wait(bar, phase)) return true;
    }
    vk_set_status(VK_ST_MBAR_TIMEOUT);
    return false;
}
// Orders what this thread has observed of shared memory in the generic proxy (other warps' ld.shared / ldmatrix reads,
// known to be over through an mbarrier) before the async-proxy operations it issues next. A producer thread executes
// it between its wait for a free stage and the bulk copy that refills the stage: the mbarrier alone orders the
// consumers' reads and the producer's wait, both in the generic proxy, but not the copy's writes, which happen in
// the async proxy (measured on B200: without the fence a refill now and then overtook a warp's last reads of the
// stage, as soon as another kernel's loads kept the memory system busy beside the GEMM).
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// global -> shared bulk copy through the TMA engine; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void tma_bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// ---------------------------------------------------------------- programmatic dependent launch
// pdl_wait: block until the kernels this one depends on have completed and their writes are visible. Everything a
// kernel does before it may only touch memory no earlier kernel of the stream writes (weights, its own smem).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Who may read what in front of its griddepcontrol.wait. A kernel can start as soon as every CTA of its predecessor
// has executed launch_dependents. The streaming GEMMs (and the two small kernels that can stand in front of a layer
// boundary: engram_gather, bf16_gemm_rows) execute it only AFTER their own wait: when their successor starts, the
// GEMM's predecessor, and with it every earlier launch, has completed, so the successor (KDA, add + norm, the layer
// boundary) may read, in front of its wait, anything written two or more launches back, just not the GEMM's output.
// All other kernels execute launch_dependents first thing: their successors are GEMMs, which read nothing but
// weights in front of their wait and should become resident as early as possible to start streaming them.
// Host: launch with the PDL attribute (the kernel must call pdl_wait before reading its predecessor's outputs).
// One-time, per-device setup at a call site (function attributes such as the opt-in to more than 48 KB of dynamic shared
// memory belong to the device's context): run(f) calls f() the first time it is reached on the current device, and again
// if f failed. Safe from several threads (f may then run more than once; it only sets attributes).
class PerDeviceOnce {
    std::atomic<bool> done_[64];

  public:
    template <class F> cudaError_t run(F f) {
        int dev = -1;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
        if (done_[dev].load(std::memory_order_acquire)) return cudaSuccess;
        e = f();
        if (e == cudaSuccess) done_[dev].store(true, std::memory_order_release);
        return e;
    }
};

bool vk_pdl_enabled();
extern long long g_vk_launches;  // kernels launched through vk_launch since the last reset (host counter)
template <typename... KArgs, typename... Args>
static inline cudaError_t vk_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = vk_pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    g_vk_launches++;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same with thread-block clusters of `cluster_x` CTAs along x (grid.x a multiple of it).
template <typename... KArgs, typename... Args>
static inline cudaError_t vk_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, int cluster_x, size_t smem,
                                            cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = vk_pdl_enabled() ? 1 : 0;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = (unsigned)cluster_x;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    g_vk_launches++;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#define VK_CUDA(call)                              \
    do {                                           \
        cudaError_t e_ = (call);                   \
        if (e_ != cudaSuccess) return (int)e_;     \
    } while (0)
