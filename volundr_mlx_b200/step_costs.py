"""What each class of kernels costs INSIDE the decode step's CUDA graph, at 1 or N tensor-parallel ranks:
`python -m volundr_mlx_b200.step_costs` or, for N ranks,
`python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m volundr_mlx_b200.step_costs`.

The 16-row ragged decode step of the synthetic 32B-shaped model (the benchmark's workload) is captured once with every
kernel, then once per class with that class's entry points left out of the graph (their launches return at once; the
step's results are then meaningless, only its duration is read). The difference to the full step is the class's
marginal cost: what the step would gain if the class were free, with the overlap between neighbouring kernels
(programmatic dependent launch) counted as it really is. Times are CUDA events around ten replays, the maximum over
ranks. One line per class: `N=<ranks> <class> <ms per step> marginal <ms> kernels <launches in the graph>`.
"""
from __future__ import annotations

import os

import numpy as np
import torch
import torch.distributed as dist

from . import _lib, batch as BT, synth
from .volundr import Model, SynthParams

CLASSES = [
    ("all", set()),
    ("no_select", {"vk_bcsa_select"}),
    ("no_prep", {"vk_attn_prep"}),
    ("no_attend", {"vk_attend_decode"}),
    ("no_gemm", {"vk_w4_gemm_xrec", "vk_w4_gemm"}),
    ("no_kda", {"vk_kda_step"}),
    ("no_attn", {"vk_attn_prep", "vk_bcsa_select", "vk_attend_decode"}),
    ("no_boundary", {"vk_mhc_boundary_ar", "vk_mhc_combine_norm_ar", "vk_mhc_mix_norm"}),
    ("no_add_rmsnorm", {"vk_add_rmsnorm_ar"}),
    ("no_silu", {"vk_silu_mul"}),
    ("no_head", {"vk_bf16_gemm_packed", "vk_argmax", "vk_argmax_pairs", "vk_argmax_merge"}),
]
CLASSES.append(("none", set().union(*(c for _, c in CLASSES))))


def context_lengths(seed=4, n=16, lo=256, hi=20000):
    """The benchmark's rows: prompts log-uniform in [256, 20000] plus a decode progress in [0, 512), seeded."""
    rng = np.random.Generator(np.random.PCG64(seed))
    prompts = np.exp(rng.uniform(np.log(lo), np.log(hi), size=n)).astype(np.int64)
    return [int(p + d) for p, d in zip(prompts, rng.integers(0, 512, size=n))]


class _Without:
    """The library with some entry points replaced by calls that do nothing and report success."""

    def __init__(self, real, skip):
        self._real, self._skip = real, skip

    def __getattr__(self, name):
        if name in self._skip:
            return lambda *a, **k: 0
        return getattr(self._real, name)


def main():
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    args = synth.volundr32b_args()
    model = Model(args, SynthParams(args, dev, seed=4, bias_mode="free"), dev, tp_rank=rank, tp_size=world, group=group)
    torch.cuda.empty_cache()
    ctx = context_lengths()
    steps_total = 400
    bc = model.make_cache(max_rows=16, n_pages=sum((c + steps_total) // 64 + 2 for c in ctx),
                          max_pages_per_row=(max(ctx) + steps_total) // 64 + 2, seed=4)
    bc.fill_synthetic(list(range(16)), ctx, seed=4)
    toks = torch.zeros(bc.B, dtype=torch.int32, device=dev)
    real = _lib.lib()
    lib_fn = _lib.lib
    BT.forward(model, bc, toks)
    base = None
    try:
        for name, skip in CLASSES:
            bc.graphs.clear()
            _lib.lib = (lambda s: (lambda: _Without(real, s)))(skip)
            for _ in range(3):
                BT.forward(model, bc, toks)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                BT.forward(model, bc, toks)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 10
            if world > 1:
                t = torch.tensor([ms], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            base = ms if base is None else base
            if rank == 0:
                print(f"N={world} {name:16s} {ms:8.3f} ms/step  marginal {base - ms:7.3f} ms  kernels {bc.kernels_per_step}", flush=True)
    finally:
        _lib.lib = lib_fn
    if world > 1:
        bc.graphs.clear()
        dist.barrier()
        torch.cuda.synchronize()
        import threading   # (tearing down the communicator can hang once peer mappings are gone: give it 20 s)

        th = threading.Thread(target=dist.destroy_process_group, daemon=True)
        th.start()
        th.join(20)
        if th.is_alive():
            os._exit(0)


if __name__ == "__main__":
    main()
