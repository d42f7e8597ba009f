// Library-wide state: the device status word and the programmatic-dependent-launch switch.
#include "common.cuh"

long long g_vk_launches = 0;

namespace {
bool g_pdl = true;
__global__ void vk_status_fetch_kernel(int* out) {
    pdl_wait();
    *out = atomicExch(&g_vk_status, 0);
}
}  // namespace

bool vk_pdl_enabled() { return g_pdl; }

extern "C" {

// 1 = launch kernels with the programmatic-stream-serialization attribute (default), 0 = plain stream order.
void vk_set_pdl(int on) { g_pdl = on != 0; }

// Copy the device status word to *device_out (device memory, 4 bytes) and clear it; stream-ordered, no sync.
int vk_status_fetch(int* device_out, cudaStream_t stream) {
    cudaError_t e = vk_launch(vk_status_fetch_kernel, dim3(1), dim3(1), 0, stream, device_out);
    return (int)e;
}

const char* vk_status_string(int code) {
    switch (code) {
        case 0: return "ok";
        case VK_ST_MBAR_TIMEOUT: return "a TMA bulk copy did not complete within the spin limit";
        case VK_ST_BAD_INDEX: return "page or block index outside its pool";
        case VK_ST_POOL_EMPTY: return "page pool exhausted";
        case VK_ST_FLAG_TIMEOUT: return "flag wait ran out";
        default: return "unknown status";
    }
}

int vk_version() { return 1; }

#ifdef VK_TRACE
int vk_trace_read(long long* host_out) {   // tuning builds only: [4096][16] cycle stamps of the traced kernel's last launch
    VK_CUDA(cudaDeviceSynchronize());
    VK_CUDA(cudaMemcpyFromSymbol(host_out, g_vk_trace, sizeof(long long) * 4096 * 16));
    return VK_OK;
}
#endif

// Kernels launched by this library since the last call with reset != 0 (a graph capture counts its kernels once).
long long vk_launch_count(int reset) {
    const long long n = g_vk_launches;
    if (reset) g_vk_launches = 0;
    return n;
}

}  // extern "C"
