/* C ABI of libvolundr_b200.so: the B200 (sm_100a) kernels of the batched ragged decode step.
 *
 * Conventions. Every pointer is a device pointer unless said otherwise. Every function that launches work takes
 * the CUDA stream last, returns 0 on success, -1 for an invalid argument found on the host, -2 for a workspace that
 * is too small, and a positive cudaError_t otherwise. Nothing here allocates, frees or synchronises unless its comment
 * says so. Device-side trouble (a bounded wait that ran out, an index outside its pool) is recorded in a status word
 * that vk_status_fetch reads.
 *
 * The reference (iggerask/volundr-mlx) has no FFI: this path sits behind Python module APIs. Each entry point below
 * names the reference function whose arithmetic it replaces (file:line in the reference repository). */
#ifndef VOLUNDR_B200_H
#define VOLUNDR_B200_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
typedef struct CUstream_st* vk_stream_t; /* == cudaStream_t */

/* ---- library state */
int vk_version(void);
/* 1 (default): kernels are launched with programmatic dependent launch, so a kernel's weight prefetch overlaps the
 * tail of its predecessor; 0: plain stream order. */
void vk_set_pdl(int on);
/* Copies the device status word to *device_out (4 bytes of device memory) and clears it. Stream-ordered. */
int vk_status_fetch(int* device_out, vk_stream_t stream);
const char* vk_status_string(int code);

/* ---- INT4 affine weight GEMM, 1..16 activation rows per pass (more rows re-stream the weights per 16).
 * Replaces nn.QuantizedLinear.__call__ -> mx.quantized_matmul(x, w, scales, biases, transpose=True, group_size, bits=4)
 * (volundr-mlx/volundr.py:185-190, 377-386, 645-648) and NaxLinear.__call__ -> qmm_nax_prepped
 * (volundr-mlx/spec/nax_hook.py:40-49, agens-mlx-bench/smallm/qmm_nax.py:128-139). */
/* Bytes of the streaming layout of an [N, K] weight. */
size_t vk_w4_packed_bytes(int N, int K);
/* Reference layout (volundr-mlx/convert.py:7-14: uint32 codes [N, K/8], nibble j of a word = element 8w + j; bf16
 * scales and biases [N, K/group], group 64 or 128) -> streaming layout. K a multiple of 64. Done once at load time. */
int vk_w4_repack(const void* w, const void* scales, const void* biases, int N, int K, int group, void* packed,
                 vk_stream_t stream);
/* bf16 out[N, K] = bf16(scale * code + bias), the exact sum rounded once: what mx.dequantize gives for the converter's
 * weights (volundr-mlx/tests/test_volundr.py:127-156). */
int vk_w4_dequant(const void* w, const void* scales, const void* biases, int N, int K, int group, void* out,
                  vk_stream_t stream);
/* Workspace bytes vk_w4_gemm needs for this shape (arrival counters + split-K partial sums). The first 16 KiB of the
 * workspace must be zero before the first call and are left zero by every call. */
size_t vk_w4_workspace_bytes(int M, int N, int K);
/* y[M, ldy] (bf16) = x[M, ldx] (bf16) . dequant(W)^T, fp32 accumulation. ldx a multiple of 8, x 16-byte aligned. */
int vk_w4_gemm(const void* packed, const void* x, int ldx, void* y, int ldy, int M, int N, int K, void* workspace,
               size_t workspace_bytes, vk_stream_t stream);
/* Testing aid: force warps per CTA (4 or 8) and the number of K slabs; 0 = choose automatically. */
void vk_w4_force_plan(int warps, int split);

#ifdef __cplusplus
}
#endif
#endif
