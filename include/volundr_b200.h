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
/* Kernels launched by the library since the last call with reset != 0 (host-side counter; a stream capture counts
 * the captured kernels once). */
long long vk_launch_count(int reset);

/* ---- INT4 affine weight GEMM. Up to 16 activation rows: one pass, two CTAs per SM (the decode step). More rows (verify
 * windows, prefill chunks) through vk_w4_gemm: passes of 64, then 32, then up to 16 rows, each streaming the weights once.
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
/* Workspace bytes vk_w4_gemm needs for this shape (arrival counters, the activation records, partial sums of ranges
 * that split a block of rows over K). The first 16 KiB of the workspace must be zero before the first call and are
 * left zero by every call (a call whose bounded wait ran out, reported through the status word, may leave a counter
 * behind: zero them again before the buffer is used by another launch). */
size_t vk_w4_workspace_bytes(int M, int N, int K);
/* y[M, ldy] (bf16) = x[M, ldx] (bf16) . dequant(W)^T, fp32 accumulation. ldx a multiple of 8, x 16-byte aligned. */
int vk_w4_gemm(const void* packed, const void* x, int ldx, void* y, int ldy, int M, int N, int K, void* workspace,
               size_t workspace_bytes, vk_stream_t stream);
/* The same product for activations that already sit in the kernel's input layout ("x records": per 64 columns 2176
 * bytes = 16 rows x 64 bf16 stored [16-byte piece][row][8 values], then the sixteen rows' sums over the group as fp32;
 * rows >= M zero). The row kernels below write this layout directly when given an `xrec_*` pointer (as the reference
 * fuses its input preparation into the producing op, agens-mlx-bench/smallm/prep_nax.py:24-148). M <= 16. */
int vk_w4_gemm_xrec(const void* packed, const void* xrec, void* y, int ldy, int M, int N, int K, void* workspace,
                    size_t workspace_bytes, vk_stream_t stream);
/* Which kernel multiplies up to 16 activation rows (vk_w4_gemm_xrec, vk_w4_gemm with M <= 16):
 *   0 (default)  mma.sync on the raw codes, scale and bias term applied per 64-column group in fp32;
 *   2, 3         the same arithmetic with the per-group products on tcgen05 (weights as the M side; the number is the
 *                steps between a warp's expansion and its accumulation of a step); differs from 0 in the last bits;
 *   4            weights dequantised to bf16 in shared memory (bit-equal to vk_w4_dequant), activations x weights on
 *                tcgen05 with the accumulator in tensor memory over all of K: the arithmetic of "dequantise, then matmul".
 * 2 .. 4 are measured slower than 0 on B200 and are kept as tested alternatives. A testing and measuring aid, global to
 * the process: set it before the first launch of a CUDA graph that records these calls. */
void vk_w4_select(int form);
/* The same streaming kernel over plain bf16 weights: the linears the reference keeps unquantised (convert.py:16-17),
 * above all lm_head (volundr.py:958, :968; batch.py:552). W [N, K] row-major bf16 is repacked once into the kernel's
 * fragment order (vk_bf16_repack); y = bf16(x . W^T), fp32 accumulation, 1..16 rows per pass. Workspace rules as for
 * vk_w4_gemm. */
size_t vk_bf16_packed_bytes(int N, int K);
int vk_bf16_repack(const void* W, int N, int K, void* packed, vk_stream_t stream);
size_t vk_bf16_workspace_bytes(int M, int N, int K);
int vk_bf16_gemm_packed(const void* packed, const void* x, int ldx, void* y, int ldy, int M, int N, int K, void* workspace,
                        size_t workspace_bytes, vk_stream_t stream);
/* The same product for many activation rows (verify windows of B x T rows, prefill chunks) on the tcgen05 tensor cores
 * with the accumulator in tensor memory: one or two tiles of 128 activation rows x 256 or 64 weight rows per CTA. The weight
 * tile is dequantised to bf16 once, bf16(s * u + b) with a single rounding (the value vk_w4_dequant gives), so results
 * differ from vk_w4_gemm by that rounding of the weights (within the bf16 bar). `packed` as for vk_w4_gemm. */
size_t vk_w4_tile_workspace_bytes(int M, int K);
/* Up to 128 rows: with a workspace of this many bytes, zeroed once by the caller (its first 16 KB hold arrival counters the
 * kernels leave at zero), the product runs split-K: every SM takes an equal range of the weight's 9216-byte steps and
 * accumulates in tensor memory, ranges that share a 256-row block add their fp32 partial sums in a fixed order; with less,
 * whole 256-row blocks per CTA, in waves. Same arithmetic either way; vk_w4_tile_split(0) forces the second form. */
size_t vk_w4_tile_workspace_bytes_n(int M, int N, int K);
void vk_w4_tile_split(int on);
int vk_w4_gemm_tile(const void* packed, const void* x, int ldx, void* y, int ldy, int M, int N, int K, void* workspace,
                    size_t workspace_bytes, vk_stream_t stream);
/* Tuning / testing aid for vk_w4_gemm_tile: weight rows per CTA (256 = a whole superblock, 64 = a quarter, for weights
 * with few rows) and tiles of 128 activation rows per CTA (1 or 2; with 2 every dequantised weight tile feeds two
 * accumulators). 0 = chosen from the shape (the default). Results do not depend on either. */
int vk_w4_tile_force(int weight_rows, int row_tiles);
/* Tuning / testing aid: force the number of persistent CTAs the work is dealt to (0 = two per SM), and the budget in
 * MB of the L2 prefetch a GEMM issues for its own weights before it waits for the kernel that produces x
 * (0 or negative = none, the default: on B200 the prefetch measured slower than none). Results do not depend on either. */
void vk_w4_force_plan(int ctas, int prefetch_mb);

/* ---- row-wise fused kernels (one CTA per token row). bf16 activations [B, D] unless noted. An `xrec_*` argument may
 * be NULL; otherwise it receives the same output as x records for a following vk_w4_gemm_xrec (B <= 16). */
/* x = embed[tok]; H[b][0..3] = x; hn = RMSNorm(x) * w_mhc0 (volundr-mlx/volundr.py:921-930, :944; batch.py:525-538).
 * With engram_prev != NULL also advances the id window [B, max(order) - 1] and hashes the n-gram rows
 * engram_rows_out [B, n_orders] (volundr.py:572-582; host ints `orders`). */
int vk_embed(const int* tok, const void* embed, const void* w_mhc0, void* H, void* hn, int* engram_prev,
             int* engram_rows_out, const int* orders, int n_orders, int engram_rows, int B, int D, float eps,
             vk_stream_t stream);
/* MHC.mix_norm (volundr.py:336-340; decode_fused.py:230-248; ops: volundr.py:264-278, :237-243): dyn linear, pre /
 * post, Sinkhorn, x_in, h = OffsetRMSNorm(x_in) * (1 + w_in). post [B,4], res [B,16] are fp32 holding bf16 values;
 * d_scratch [B, 24] fp32 receives the dyn linear's output. */
int vk_mhc_mix_norm(const void* H, const void* hn, const void* w_dyn, const void* pre_s, const void* post_s,
                    const void* res_s, const void* w_in, void* x_in, void* h, void* xrec_h, float* post, float* res,
                    float* d_scratch, int B, int D, int iters, float eps, vk_stream_t stream);
/* kernels.rms_norm(x, w, eps, offset, r) (kernels.py:285-306; volundr.py:893-899): h2 = bf16(x + r) (r, h2 may be
 * NULL), hn = RMSNorm(h2) * (offset + w). */
/* (With r given, x is read before the kernel waits for the launch in front of it: that launch may write r, not x.) */
int vk_add_rmsnorm(const void* x, const void* r, const void* w, void* h2, void* hn, void* xrec_hn, int B, int D, float eps,
                   int offset, vk_stream_t stream);
/* _silu_mul (volundr.py:166-168) on gu = [gate (I) | up (I)] rows of stride ld_gu. */
int vk_silu_mul(const void* gu, void* act, void* xrec_act, int B, int I, int ld_gu, vk_stream_t stream);
/* Engram row gather + RMSNorm (volundr.py:594-595). tables / ld_table / col0 are host arrays of n_orders entries. */
int vk_engram_gather(const void* const* tables, const int* ld_table, const int* col0, const int* rows, const void* w,
                     void* e, int B, int n_orders, int dim, float eps, vk_stream_t stream);
/* Residual add + (Engram gate) + MHC.combine_norm (volundr.py:342-347, :281-290, :594-597; decode_fused.py:341-355):
 * H updated in place; hn = next layer's mHC norm of the stream mean, or with final_norm the model's final norm of
 * stream 0 (volundr.py:949). */
int vk_mhc_combine_norm(void* H, const void* h2, const void* m, const void* x_in, const float* post, const float* res,
                        const void* w_next, void* hn, const void* eng_val, const void* eng_gate_w, const void* eng_gate_b,
                        void* y_out, int B, int D, int final_norm, float eps, vk_stream_t stream);
/* vk_mhc_combine_norm of layer i and vk_mhc_mix_norm of layer i + 1 in one launch (VolundrModel._fused_layers runs them
 * back to back, volundr.py:945-948): H, x_in, post, res are updated in place for the next layer; h / xrec_h receive its
 * input norm. Same values as the two separate calls. D / 8 <= 640. */
void vk_mhc_boundary_set_cluster(int on);   /* 1: four CTAs (one cluster) per row when D % 1024 == 0; 0 (default): one */
int vk_mhc_boundary(void* H, const void* h2, const void* m, void* x_in, float* post, float* res, const void* w_next,
                    const void* eng_val, const void* eng_gate_w, const void* eng_gate_b, const void* w_dyn, const void* pre_s,
                    const void* post_s, const void* res_s, const void* w_in, void* h, void* xrec_h, int B, int D, int iters,
                    float eps, vk_stream_t stream);
/* The linears kept in bf16 (convert.py:16-17): y = bf16(x . W^T + bias), W [N, K] row-major. */
int vk_bf16_gemm(const void* x, int ldx, const void* W, const void* bias, void* y, int ldy, int M, int N, int K,
                 vk_stream_t stream);
/* Greedy token: first maximum over logits[:, :valid] (scheduler.py:391). */
int vk_argmax(const void* logits, int ld, int valid, int* out, int B, vk_stream_t stream);
/* The same over a vocabulary split across tensor-parallel ranks (no counterpart in the single-GPU reference): each rank
 * writes pairs [B, 2] = (float bits of its largest logit among its first `valid` columns, index_offset + its first
 * position; (-inf, INT_MAX) when valid <= 0); after an all-gather to [ranks, B, 2], vk_argmax_merge picks the largest
 * value, ties to the lowest index. */
int vk_argmax_pairs(const void* logits, int ld, int valid, int index_offset, int* pairs, int B, vk_stream_t stream);
int vk_argmax_merge(const int* pairs, int n_ranks, int* out, int B, vk_stream_t stream);

/* ---- Tensor-parallel exchange inside the consuming kernel (no counterpart in the single-GPU reference). The ranks of
 * one node hold partial products of the row-parallel linears (out_proj / o_proj, down_proj). Instead of a separate
 * all-reduce, the kernel that consumes the sum (vk_add_rmsnorm_ar, vk_mhc_boundary_ar, vk_mhc_combine_norm_ar: one CTA
 * per row) pushes its partial row into every peer's region with peer stores (every 8-byte unit = 4 bytes of data + the
 * call's sequence number, so neither a fence nor a flag follows), polls (bounded) its own region until the peers'
 * units carry that number and adds the rows in rank order; the bf16 sum replaces the partial row in `r` / `m`, which is
 * therefore not const. Set-up per rank: vk_ar_alloc a region of vk_ar_region_bytes, pass the 64-byte handle to the
 * other ranks (any host channel), vk_ar_open theirs, vk_ar_fill the descriptor, synchronise the ranks once (host
 * barrier) before the first step. Per step: `call` = 0 .. calls_per_step - 1 in the same order on every rank, then
 * vk_ar_advance once. A wait that runs out sets status 4 (vk_status_fetch) and the step's results are invalid.
 * A null descriptor, or world 1, means no exchange: the _ar entry points then equal the plain ones. */
typedef struct vk_ar_desc {
    int world, rank, rows, row_elems, calls_per_step;
    unsigned spin_limit;   /* polls (>= 100 ns each) before a wait gives up; vk_ar_fill sets a default of seconds */
    void* slots[8];
    int* step;
} vk_ar_desc;
size_t vk_ar_region_bytes(int world, int rows, int D);   /* 0: unsupported (world <= 8, D a multiple of 8) */
int vk_ar_alloc(size_t bytes, void** ptr, void* handle64);
int vk_ar_open(const void* handle64, void** ptr);
int vk_ar_close(void* ptr);
int vk_ar_free(void* ptr);
int vk_ar_fill(vk_ar_desc* d, int world, int rank, int rows, int D, int calls_per_step, void* const* bases);
int vk_ar_advance(const vk_ar_desc* d, vk_stream_t stream);
int vk_add_rmsnorm_ar(const void* x, void* r, const void* w, void* h2, void* hn, void* xrec_hn, int B, int D, float eps,
                      int offset, const vk_ar_desc* ar, int call, vk_stream_t stream);
int vk_mhc_combine_norm_ar(void* H, const void* h2, void* m, const void* x_in, const float* post, const float* res,
                           const void* w_next, void* hn, const void* eng_val, const void* eng_gate_w, const void* eng_gate_b,
                           void* y_out, int B, int D, int final_norm, float eps, const vk_ar_desc* ar, int call,
                           vk_stream_t stream);
int vk_mhc_boundary_ar(void* H, const void* h2, void* m, void* x_in, float* post, float* res, const void* w_next,
                       const void* eng_val, const void* eng_gate_w, const void* eng_gate_b, const void* w_dyn, const void* pre_s,
                       const void* post_s, const void* res_s, const void* w_in, void* h, void* xrec_h, int B, int D, int iters,
                       float eps, const vk_ar_desc* ar, int call, vk_stream_t stream);

/* ---- Kimi Delta Attention decode step (KDA.__call__, volundr.py:388-410: DF.kda_conv_gates decode_fused.py:469-493,
 * kernels.gated_delta_vec kernels.py:446-458, kernels.gated_norm kernels.py:918-928, plus in_proj_b and f_up).
 * proj [B, ldp] = [q | k | v | z (at off_z) | f_down (at off_fd)]; conv [2, slots, 3, C] with *parity naming the
 * current buffer; S fp32 [slots, HV, 128, 128] updated in place; out [B, HV*128]. */
/* w_fup of vk_kda_step is f_up.weight [HV*128, rank] repacked once at load time to [HV][rank / 8][128][8]. */
int vk_kda_pack_fup(const void* src, void* dst, int HV, int rank, vk_stream_t stream);
int vk_kda_configure(void);   /* once per device, outside stream capture: shared-memory carve-out hint for vk_kda_step */
int vk_kda_step(const void* proj, int ldp, int off_z, int off_fd, const void* h, const void* w_b, const void* w_fup,
                const float* conv_w, const float* A_log, const float* dt_bias, const void* norm_w, void* conv,
                const int* parity, size_t conv_stride, float* S, void* out, void* xrec_out, int B,
                int D, int Hk, int HV, int Dk, int Dv, int rank, float eps, vk_stream_t stream);
/* The same recurrence over a chunk of T tokens per row in one launch, the state read and written once: the prefill
 * form (kernels.gated_delta_tg, kernels.py:544-555) and the verify / commit-replay form (verify._kda,
 * spec/verify.py:33-53; batch_spec.py:186-195). Rows of proj / h / out are b * T + t. accept (optional, [B]): row b
 * stops after accept[b] tokens; later tokens leave state, conv window and output alone. Results equal T (or accept[b])
 * calls of vk_kda_step bit for bit. The conv window after the chunk lands in the other buffer, as after one step: flip
 * the parity word once per launch. */
int vk_kda_chunk(const void* proj, int ldp, int off_z, int off_fd, const void* h, const void* w_b, const void* w_fup,
                 const float* conv_w, const float* A_log, const float* dt_bias, const void* norm_w, void* conv,
                 const int* parity, size_t conv_stride, float* S, void* out, const int* accept, int write_state, int B, int T,
                 int D, int Hk, int HV, int Dk, int Dv, int rank, float eps, vk_stream_t stream);
/* (write_state = 0: outputs only; the state and the conv buffers are not touched and the parity word is not to be
 * flipped: the verify pass in front of a commit.) */
/* Ragged chunks: request b has accept[b] <= T tokens of its own and its rows of proj / h / out start at
 * row_offset[b] (the requests' rows lie one after another, nothing is padded); row_offset null = vk_kda_chunk. */
int vk_kda_chunk_ragged(const void* proj, int ldp, int off_z, int off_fd, const void* h, const void* w_b, const void* w_fup,
                        const float* conv_w, const float* A_log, const float* dt_bias, const void* norm_w, void* conv,
                        const int* parity, size_t conv_stride, float* S, void* out, const int* accept,
                        const int* row_offset, int write_state, int B, int T, int D, int Hk, int HV, int Dk, int Dv,
                        int rank, float eps, vk_stream_t stream);
/* h, the state S, both conv buffers and the parity word are read before the kernel waits for the launch in front of
 * it (they stream in while that launch finishes): none of them may be written by that launch. proj may. */

/* ---- paged ragged attention (64-token pages). */
typedef struct vk_attn_geom {
    int Hq, KVH, D;        /* heads of this shard, head dim (128) */
    int W, C, topk;        /* BCSA window, block size, far blocks kept; W = 0: dense causal attention */
    int IH, Di;            /* indexer heads / dim (indexer mode) */
    int NS;                /* selection groups: 1 = shared indexer (reference), KVH = per kv head from pooled keys */
    int far_tokens;        /* 1: far keys are the tokens of the chosen blocks, 0: their mean-pooled K/V (reference) */
    int max_pages, n_pages;
} vk_attn_geom;
/* BatchRows / BCSAStep (batch.py:52-122) on the GPU: allocates a page from free_list[--*free_top] for every row whose
 * next position opens one (rows in order) and writes desc [B, 8] = {pos, page, row in page, closes a block, nv, nf,
 * keys attended, window start}. */
int vk_batch_step_begin(const int* pos, int* table, int max_pages, int* free_list, int* free_top, int* desc, int B, int W,
                        int C, int topk, vk_stream_t stream);
/* The same allocation for a chunk of tokens per row (the verify window of batch_spec.verify_forward, batch_spec.py:107-158;
 * a prefill chunk of session.prefill_iter, session.py:351-387): row b is about to hold positions pos[b] ..
 * pos[b] + lens[b] - 1 and every position that starts a page takes one, rows in order. */
int vk_pages_open(const int* pos, const int* lens, int* table, int max_pages, const int* free_list, int* free_top, int B,
                  vk_stream_t stream);
/* Pages back to the pool without a host round trip: item i returns the table entries [first[i], last[i]) of row rows[i]
 * (device arrays of n ints), ascending, or descending with `reverse`; the entries become -1. Used when a commit keeps
 * fewer tokens than the verify pass opened pages for (batch_spec.commit, batch_spec.py:173-199) and when a row leaves
 * the batch (BatchCache.apply, batch.py:416-431). */
int vk_pages_release(const int* rows, const int* first, const int* last, int n, int reverse, int* table, int max_pages,
                     int* free_list, int* free_top, int n_pages, vk_stream_t stream);
/* BatchRows.advance (batch.py:74-77): pos += 1; flips *parity. */
int vk_batch_step_end(int* pos, int* parity, int B, vk_stream_t stream);
/* Attention._batched up to the cache write (volundr.py:737-747; batch.py:224-259): q/k offset norms, RoPE at pos[b],
 * K/V into the row's page, indexer query/key norms, and the pooled means of a block the step closes. */
int vk_attn_prep(const vk_attn_geom* g, const void* proj, int ldp, int off_k, int off_v, const void* idxq, const void* idxk,
                 const void* q_norm, const void* k_norm, const void* idx_norm, const int* pos, const int* table, void* q,
                 void* qi, void* K, void* V, void* PK, void* PV, void* BK, void* IK, int B, int rope_dims, double rope_theta,
                 float eps, vk_stream_t stream);
/* vk_attn_prep for rows that are consecutive positions of one sequence (a verify window, a prefill chunk): a block may
 * then be closed by a position whose neighbours other rows of the same launch write, so all rows are written first
 * (mode 1) and pooled by a second launch (mode 2); mode 0 = vk_attn_prep. row_map (optional, [B]): the cache row whose
 * open-block indexer keys (IK) a row shares. */
int vk_attn_prep_rows(const vk_attn_geom* g, const void* proj, int ldp, int off_k, int off_v, const void* idxq, const void* idxk,
                      const void* q_norm, const void* k_norm, const void* idx_norm, const int* pos, const int* table, void* q,
                      void* qi, void* K, void* V, void* PK, void* PV, void* BK, void* IK, int B, int rope_dims,
                      double rope_theta, float eps, int mode, const int* row_map, vk_stream_t stream);
/* vk_attn_prep_rows for the shared-indexer form of BCSA: the C-slot ring of open-block indexer keys cannot hold a chunk
 * that spans more than one block, so the rows' normed indexer keys go to ikc [B, Di] instead, and a block that closes
 * inside the chunk is pooled from them (plus the ring for positions in front of first_pos[b], the first position the
 * chunk brought for row b's sequence), as BCSACache.update pools from `ci = ik_open ++ chunk keys`
 * (batch_spec.py:140-158, volundr.py:508-533). The ring is left untouched; the caller stores the open block's keys of
 * the tokens it keeps. ikc null: vk_attn_prep_rows. */
int vk_attn_prep_chunk(const vk_attn_geom* g, const void* proj, int ldp, int off_k, int off_v, const void* idxq, const void* idxk,
                       const void* q_norm, const void* k_norm, const void* idx_norm, const int* pos, const int* table, void* q,
                       void* qi, void* K, void* V, void* PK, void* PV, void* BK, void* IK, int B, int rope_dims,
                       double rope_theta, float eps, int mode, const int* row_map, void* ikc, const int* first_pos,
                       vk_stream_t stream);
/* _block_scores + _topk_blocks (volundr.py:601-618; kernels.bcsa_scores kernels.py:1227-1240, bcsa_topk :86-98):
 * sel [B, NS, topk] ascending block indices (-1 padded), nsel [B, NS]. scratch: max_blocks uint32 per (row, group). */
int vk_attn_configure(void);   /* once per device, outside stream capture: shared-memory opt-in of the selection kernel
                                * (the first vk_bcsa_select on a device does the same) */
size_t vk_bcsa_select_scratch_bytes(const vk_attn_geom* g, int B, int max_blocks);
int vk_bcsa_select(const vk_attn_geom* g, const void* q, const void* keys, const int* pos, const int* table, void* scratch,
                   int max_blocks, int* sel, int* nsel, int B, vk_stream_t stream);
/* Far-block selection for callers that may not allocate device memory: a CUDA-graph node builder, a plugin running
 * inside another runtime's memory budget, or a process whose allocator is owned by someone else has no buffer to hand
 * in as `scratch`. This variant has no counterpart in the reference. It computes exactly what vk_bcsa_select computes
 * but keeps the sort keys in a 1 MiB array that is part of the library image, so it calls no cudaMalloc / cudaFree
 * and no allocating library routine. Limits: B <= 16 rows, NS <= 8 groups, max_pages * (64 / C) <= 2048 blocks per
 * row; anything larger returns -3 (VK_ETOOBIG) and launches nothing. The first call on each device looks up the
 * array's device address (cudaGetSymbolAddress, with that device current): make that first call outside any stream
 * capture. All calls on a device share the one array, which keeps whatever the last call left in it (nothing in it
 * needs clearing: every key is written before it is read): two calls that overlap on the GPU (different streams, or
 * a graph replayed concurrently) race on it. */
int vk_bcsa_select_static(const vk_attn_geom* g, const void* q, const void* keys, const int* pos, const int* table, int* sel,
                          int* nsel, int B, vk_stream_t stream);
/* The SDPA of _bcsa_batched / BatchKVCache.attend (volundr.py:790-791; batch.py:315-316) over window pages and far
 * keys, split over `nsplit` CTAs per (row, kv head), merged, times sigmoid(gate) (volundr.py:177-179).
 * part: fp32 scratch of vk_attend_scratch_bytes. out [B, Hq*D]. */
size_t vk_attend_scratch_bytes(const vk_attn_geom* g, int B, int nsplit);
/* 1 (default): Q K^T and P V on the tensor cores (bf16 probabilities); 0: the scalar fp32 kernel, kept as a cross-check. */
void vk_attend_set_tensor_cores(int on);
int vk_attend_decode(const vk_attn_geom* g, const void* q, const void* K, const void* V, const void* PK, const void* PV,
                     const int* pos, const int* table, const int* sel, const int* nsel, const void* proj, int ldp,
                     void* part, int nsplit, void* out, void* xrec_out, int B, vk_stream_t stream);

/* The same attention for rows that are consecutive positions of one sequence (the T tokens of a verify window, a
 * prefill chunk): bcsa_verify.attend (bcsa_verify.py:278-317), far_union + bcsa_attend (kernels.py:931-1020, :1023-1165;
 * volundr.py:793-827) and the dense layer of batch_spec._dense (batch_spec.py:50-64). Rows are given in tiles of up to
 * 16 consecutive rows of one sequence (tile_first / tile_count, device arrays of n_tiles ints; the rows' positions are
 * pos[first], pos[first] + 1, ...): a tile's K / V are read once for all its rows, far blocks = the union of the rows'
 * selections with a per-row mask. K / V of every row must already be in the pages (vk_attn_prep_chunk). nv_cap: an upper
 * bound of the valid far blocks of any row (sizes the kernel's shared memory: vk_attend_chunk_smem_bytes; more than about
 * 200 KB returns -3 and the caller uses vk_attend_decode). part: as for vk_attend_decode with B = R. */
size_t vk_attend_chunk_smem_bytes(const vk_attn_geom* g, int nv_cap);
int vk_attend_chunk(const vk_attn_geom* g, const void* q, const void* K, const void* V, const void* PK, const void* PV,
                    const int* pos, const int* table, const int* sel, const int* nsel, const int* tile_first,
                    const int* tile_count, int n_tiles, int nv_cap, const void* proj, int ldp, void* part, int nsplit, void* out,
                    int R, vk_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
