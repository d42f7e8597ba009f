// One-shot all-reduce of a few activation rows across the GPUs of one node, done INSIDE the kernel that consumes the
// sum (the residual add + norm after out_proj / o_proj, the layer-boundary kernel after down_proj). Tensor-parallel
// ranks hold partial products of the row-parallel linears; the reference is single-GPU and has no counterpart.
//
// Every rank owns one region of device memory that all ranks have mapped (CUDA IPC):
//     header                            the local step counter
//     slots [4][world][rows][D] lines   slots[seq & 3][src][b] = the partial row that `src` pushed, as 8-byte units
//                                       {two bf16 of data, the push's sequence number}: 16-byte lines of two units
// The sequence number travels WITH the data, so a push needs neither a fence nor a separate flag, and the receiver
// needs one NVLink crossing, not a store + acknowledged fence + flag: the CTA that owns (a part of) row b
// (1) stores its partial row into every peer's slots[.][me][b], one 16-byte volatile store per line (an aligned
//     8-byte unit is never torn, so data and number of a unit arrive together),
// (2) polls - bounded - its own slots[.][p][b] for every peer p until both units of a line carry this call's number
//     (a slot still holds the number of four calls ago until the new line lands),
// (3) adds the `world` partial rows in rank order in fp32 (the same order on every rank: all ranks get the same bits)
//     and leaves the bf16 sum in its local row.
// The sequence number is step * calls_per_step + call + 1 with `step` a device counter that vk_ar_advance bumps once
// per decode step, so a captured CUDA graph can be replayed. A rank pushes call k + 1 only after it has read every
// peer's lines of call k, and a peer can push call k + 4 into the same slot only after it has read this rank's lines
// of calls k + 1 .. k + 3, which this rank pushes after reading call k: a line is never overwritten before it is read.
// A wait that runs out sets VK_ST_FLAG_TIMEOUT and returns (the sum is then wrong, the host sees the status); once
// the status word is set, later waits give up at once, so a lost peer costs one time-out and not one per call.
#pragma once
#include "common.cuh"

constexpr int kArMaxWorld = 8;
constexpr int kArSlots = 4;
constexpr int kArParts = 4;     // a row may be exchanged in up to four independent parts (one CTA each)
constexpr uint32_t kArSpinDefault = 1u << 23;   // polls of >= 100 ns each: several seconds, to ride out host-side skew

// The caller's descriptor (public header: vk_ar_desc). Pointers of rank p are that rank's region as mapped into this
// process (vk_ar_open), offset by vk_ar_fill.
typedef struct vk_ar_desc {
    int world, rank, rows, row_elems, calls_per_step;
    unsigned spin_limit;           // polls before a wait gives up (vk_ar_fill sets the default)
    void* slots[8];
    int* step;
} vk_ar_desc;

struct VkArDesc {              // what the kernels get
    int world, rank, rows, calls_per_step;
    uint32_t spin_limit;
    uint8_t* slots[kArMaxWorld];   // slots[p]: base of rank p's slot array (slots[rank] is local)
    int* step;                     // local step counter
};

struct VkArCall {              // kernel argument: descriptor + which call of the step this is (world <= 1: no exchange)
    VkArDesc d;
    int call;
};

__device__ __forceinline__ size_t ar_slot_off(const VkArDesc& d, int slot, int src, int b, int D) {
    return ((((size_t)slot * d.world + src) * d.rows + b) * (size_t)D) * 4;   // (lines: twice the bf16 bytes)
}

// All threads of the CTA that owns part `part` of `nparts` (<= kArParts) equal parts of row b call this after
// griddepcontrol.wait. `row` = the rank's partial [D] bf16 in local memory; on return the part holds the sum over ranks.
// (D / nparts) % 8 == 0. Every part has its own flag word, so the CTAs of a row need not wait for one another.
__device__ __forceinline__ void ar_reduce_span(const VkArCall& a, __nv_bfloat16* row, int b, int D, int part, int nparts);
__device__ __forceinline__ void ar_reduce_row(const VkArCall& a, __nv_bfloat16* row, int b, int D) {
    ar_reduce_span(a, row, b, D, 0, 1);
}
__device__ __forceinline__ void ar_reduce_span(const VkArCall& a, __nv_bfloat16* row, int b, int D, int part, int nparts) {
    const VkArDesc& d = a.d;
    if (d.world <= 1) return;
    const uint32_t seq = (unsigned)*reinterpret_cast<volatile int*>(d.step) * (unsigned)d.calls_per_step + (unsigned)a.call + 1u;
    const int slot = (int)(seq & (kArSlots - 1));
    const int nvec_part = (D / nparts) >> 3;
    const int v_begin = part * nvec_part, nvec = v_begin + nvec_part;
    uint4* rowv = reinterpret_cast<uint4*>(row);
    // (1) push: every 16 bytes of the row become two lines {w0, seq, w1, seq}, {w2, seq, w3, seq} in every peer's region
    for (int v = v_begin + threadIdx.x; v < nvec; v += blockDim.x) {
        const uint4 val = rowv[v];
        for (int p = 0; p < d.world; p++) {
            if (p == d.rank) continue;
            uint4* dst = reinterpret_cast<uint4*>(d.slots[p] + ar_slot_off(d, slot, d.rank, b, D)) + 2 * (size_t)v;
            asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %2};" ::"l"(dst), "r"(val.x), "r"(seq), "r"(val.y) : "memory");
            asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %2};" ::"l"(dst + 1), "r"(val.z), "r"(seq), "r"(val.w) : "memory");
        }
    }
    // (2) + (3): the same thread polls the lines of its own vectors (the peers' threads of the same index push them)
    uint32_t budget = *reinterpret_cast<volatile int*>(&g_vk_status) == 0 ? d.spin_limit : 0u;
    bool ok = true;
    const uint8_t* local = d.slots[d.rank];
    for (int v = v_begin + threadIdx.x; v < nvec; v += blockDim.x) {
        float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int p = 0; p < d.world; p++) {
            uint4 u;
            if (p == d.rank) {
                u = rowv[v];
            } else {
                const uint4* src = reinterpret_cast<const uint4*>(local + ar_slot_off(d, slot, p, b, D)) + 2 * (size_t)v;
                uint4 l0, l1;
                uint32_t polls = 0;
                for (;;) {
                    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(l0.x), "=r"(l0.y), "=r"(l0.z), "=r"(l0.w) : "l"(src) : "memory");
                    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(l1.x), "=r"(l1.y), "=r"(l1.z), "=r"(l1.w) : "l"(src + 1) : "memory");
                    if (l0.y == seq && l0.w == seq && l1.y == seq && l1.w == seq) break;
                    if (budget == 0) { ok = false; break; }   // give up: the host will see the status
                    budget--;
                    if (++polls > 32) __nanosleep(100);
                }
                u = make_uint4(l0.x, l0.z, l1.x, l1.z);
            }
            s[0] += bf_lo(u.x); s[1] += bf_hi(u.x); s[2] += bf_lo(u.y); s[3] += bf_hi(u.y);
            s[4] += bf_lo(u.z); s[5] += bf_hi(u.z); s[6] += bf_lo(u.w); s[7] += bf_hi(u.w);
        }
        uint4 o;
        o.x = pack_bf2(s[0], s[1]); o.y = pack_bf2(s[2], s[3]); o.z = pack_bf2(s[4], s[5]); o.w = pack_bf2(s[6], s[7]);
        rowv[v] = o;
    }
    if (!ok) vk_set_status(VK_ST_FLAG_TIMEOUT);
    __syncthreads();
}
