// Host side of the in-kernel all-reduce (allreduce.cuh): the per-rank region, its CUDA IPC handle, the descriptor.
// No counterpart in the reference (single GPU).
#include "allreduce.cuh"

namespace {

__global__ void ar_advance_kernel(int* step) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) *step = *step + 1;
}

constexpr size_t kArHeader = 4096;   // the step counter lives in the region's first 4 KB (its last 64 bytes)

inline size_t ar_slots_bytes(int world, int rows, int D) { return (size_t)kArSlots * world * rows * D * 4; }

}  // namespace

extern "C" {

size_t vk_ar_region_bytes(int world, int rows, int D) {
    if (world < 1 || world > kArMaxWorld || rows < 1 || D < 8 || D % 8 != 0) return 0;
    return kArHeader + ar_slots_bytes(world, rows, D);
}

// cudaMalloc'ed (IPC needs a plain allocation), zeroed region + its 64-byte IPC handle for the other ranks.
int vk_ar_alloc(size_t bytes, void** ptr, void* handle64) {
    if (bytes == 0 || ptr == nullptr || handle64 == nullptr) return VK_EINVAL;
    void* p = nullptr;
    VK_CUDA(cudaMalloc(&p, bytes));
    VK_CUDA(cudaMemset(p, 0, bytes));
    VK_CUDA(cudaDeviceSynchronize());
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) { cudaFree(p); return (int)e; }
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(handle64, &h, 64);
    *ptr = p;
    return VK_OK;
}

int vk_ar_open(const void* handle64, void** ptr) {
    if (handle64 == nullptr || ptr == nullptr) return VK_EINVAL;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    VK_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return VK_OK;
}

int vk_ar_close(void* ptr) {
    VK_CUDA(cudaIpcCloseMemHandle(ptr));
    return VK_OK;
}

int vk_ar_free(void* ptr) {
    VK_CUDA(cudaFree(ptr));
    return VK_OK;
}

// bases[p] = rank p's region as mapped here (bases[rank] = the local allocation).
int vk_ar_fill(vk_ar_desc* d, int world, int rank, int rows, int D, int calls_per_step, void* const* bases) {
    if (d == nullptr || bases == nullptr || vk_ar_region_bytes(world, rows, D) == 0 || rank < 0 || rank >= world ||
        calls_per_step < 1)
        return VK_EINVAL;
    *d = vk_ar_desc{};
    d->world = world; d->rank = rank; d->rows = rows; d->row_elems = D; d->calls_per_step = calls_per_step;
    d->spin_limit = kArSpinDefault;
    for (int p = 0; p < world; p++) {
        if (bases[p] == nullptr) return VK_EINVAL;
        d->slots[p] = (uint8_t*)bases[p] + kArHeader;
    }
    d->step = (int*)((uint8_t*)bases[rank] + kArHeader - 64);
    return VK_OK;
}

// Once per decode step, after the step's last exchange: the next step's sequence numbers.
int vk_ar_advance(const vk_ar_desc* d, cudaStream_t stream) {
    if (d == nullptr || d->step == nullptr) return VK_EINVAL;
    return (int)vk_launch(ar_advance_kernel, dim3(1), dim3(32), 0, stream, d->step);
}

}  // extern "C"
