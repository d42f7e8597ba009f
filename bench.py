"""Benchmark of the batched ragged decode step: 16 requests on the 72-layer 32B-shaped W4 model.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

Prints ONE JSON line (rank 0). `value` = decode tokens per second over all rows with inputs resident on the device
(the step replayed as a CUDA graph, greedy tokens fed back on the device); `e2e` = the same through the public batch
API with the step's tokens coming from pinned host memory and the greedy ids read back every step; `roofline` = the
W4 GEMM kernel (the dominant kernel) timed alone over every weight of the model; `cpu_baseline` = the CPU oracle timed
on a bounded sample. With N > 1 (torchrun) the model is sharded tensor-parallel over the ranks.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "batched decode tok/s (16 ragged reqs, 32B-shaped W4)"
B_ROWS = 16
# dram__bytes_read.sum + dram__bytes_write.sum of w4_gemm_kernel over its algorithmic bytes, from the ncu captures
# summarised in profiles/w4_gemm_m16_ncu.txt, weighted by the two shapes' bytes
NCU_TRAFFIC_RATIO = 1.02


def measured_peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def context_lengths(seed=4, n=B_ROWS, lo=256, hi=20000):
    """Prompt lengths log-uniform in [256, 20000], plus a decode progress uniform in [0, 512) (seeded)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    prompts = np.exp(rng.uniform(np.log(lo), np.log(hi), size=n)).astype(np.int64)
    return [int(p + d) for p, d in zip(prompts, rng.integers(0, 512, size=n))]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.t.join(timeout=2)
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i].lower().startswith("active")})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ CPU baseline
SAMPLE_LAYERS = 2     # layers of the bounded CPU sample (1 KDA + 1 BCSA, full width)
SAMPLE_SCALE = 36     # 72 layers / 2; the sample also holds 1/36 of the lm_head rows


def host_threads():
    """All host cores for the CPU arm, set explicitly: NumPy's BLAS does not follow torch.set_num_threads, and under
    torchrun the environment carries OMP_NUM_THREADS=1, which the BLAS read when it was loaded."""
    cores = os.cpu_count() or 1
    try:
        cores = len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        pass
    try:
        from threadpoolctl import threadpool_limits

        threadpool_limits(limits=cores)
    except Exception:      # threadpoolctl missing: the BLAS keeps the thread count it was loaded with
        pass
    try:
        import torch

        torch.set_num_threads(cores)
    except Exception:
        pass
    return cores


def cpu_rows(orc, a, ctx, seed=4):
    """Oracle rows that already hold the GPU arm's contexts: K/V ~ N(0, 1) (bf16 values) by position, block means pooled
    from them, KDA state ~ N(0, 0.1), conv window ~ N(0, 1): the distributions BatchCache.fill_synthetic draws."""
    from oracle.numerics import bf

    rng = np.random.Generator(np.random.PCG64(seed))
    rows = []
    KVH, D, C = a.num_key_value_heads, a.head_dim, a.bcsa_compress
    for P in ctx:
        r = orc.new_row()
        r.pos = int(P)
        for i, m in enumerate(a.mixer_types):
            st = r.layers[i]
            if m == "kda":
                st["conv"] = bf(rng.normal(0, 1, size=st["conv"].shape))
                st["S"] = rng.normal(0, 0.1, size=st["S"].shape).astype(np.float32)
                continue
            K = bf(rng.standard_normal(size=(P, KVH, D), dtype=np.float32))
            V = bf(rng.standard_normal(size=(P, KVH, D), dtype=np.float32))
            st["k"], st["v"] = list(K), list(V)
            if m == "bcsa":
                nb = P // C
                st["pk"] = list(bf(K[: nb * C].reshape(nb, C, KVH, D).sum(1) * np.float32(1.0 / C)))
                st["pv"] = list(bf(V[: nb * C].reshape(nb, C, KVH, D).sum(1) * np.float32(1.0 / C)))
        rows.append(r)
    return rows


def cpu_sample(steps, warmup=1, rows=B_ROWS):
    """The CPU oracle on a bounded sample of the workload: 2 of the 72 layers (1 KDA + 1 BCSA) at full width plus 1/36
    of the lm_head, the 16 rows at the GPU arm's contexts. Every step is really run and timed; returns the measured
    seconds per sample step and the tokens per second of the whole model derived from it (x 36 layers' worth)."""
    from oracle.model import Oracle
    from volundr_mlx_b200 import synth

    cores = host_threads()
    a = synth.volundr32b_args(num_hidden_layers=SAMPLE_LAYERS, mixer_types=["kda", "bcsa"], engram_layers=[],
                              vocab_size=4224, vocab_valid=4224, engram_rows=1024)
    p = synth.make_params(a, seed=4, quant=True, bias_mode="free")
    orc = Oracle(a, p, exact=False, fast=True)
    ctx = context_lengths()[:rows]
    rws = cpu_rows(orc, a, ctx)
    rng = np.random.default_rng(4)
    for _ in range(max(1, warmup)):  # untimed: the first one also builds the weight cache
        for r in rws:
            orc.step(r, int(rng.integers(0, a.vocab_valid)))
    t0 = time.perf_counter()
    for _ in range(steps):
        for r in rws:
            orc.step(r, int(rng.integers(0, a.vocab_valid)))
    dt = (time.perf_counter() - t0) / steps
    toks = rows / (dt * SAMPLE_SCALE)
    return {"value": toks, "unit": "tok/s", "cores": cores, "kind": "port", "sample_step_s": dt, "sample_steps": steps,
            "sample": f"{steps} timed steps x {rows} rows (ctx {min(ctx)}..{max(ctx)}) of {SAMPLE_LAYERS}/72 layers (1 KDA + 1 BCSA, "
                      f"full width) + 1/{SAMPLE_SCALE} lm_head; value = {rows} rows / ({SAMPLE_SCALE} x measured seconds per sample step)"}


def run_reference(a):
    """--impl reference: the reference's MLX CPU path cannot run here (mlx is not installed and cannot be), so the CPU
    restatement of that path (oracle/) is what is timed, on all host threads. A step of this arm is one step of the
    bounded sample (2 of the 72 layers + 1/36 of the lm_head, 16 rows): `steps`, `warmup` and `ms_per_step` are what was
    really run and measured; only `value` carries the x 36 to the whole model."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    base = cpu_sample(steps=a.steps, warmup=a.warmup)
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": "tok/s", "n_gpus": a.gpus, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": 1e3 * base["sample_step_s"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "volundr-32b-shaped W4 g64, 16 ragged rows, decode step; one step here = the bounded CPU "
                                   f"sample ({SAMPLE_LAYERS} of 72 layers + 1/{SAMPLE_SCALE} lm_head), value scaled x{SAMPLE_SCALE} "
                                   "to the whole model",
                       "reference": "MLX CPU path unavailable on this box (mlx not installable); CPU restatement timed"},
            "cpu_baseline": base, "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "wall_s": time.perf_counter() - t0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ GPU arm
def gemm_roofline(model, bc, torch, ops, reps=3):
    """Every W4 GEMM of one step, launched back to back over all layers' weights (18+ GB: far beyond L2), timed with
    CUDA events on the launching stream. Returns (launches per step, algorithmic bytes per launch, seconds per launch)."""
    from volundr_mlx_b200 import _lib

    L = _lib.lib()
    B = bc.B
    jobs = []
    for w in model.layers:
        for nm, xr, y in (("proj", bc.xr_h, bc.proj), ("out", bc.xr_mix, bc.r), ("gate_up", bc.xr_hn2, bc.gu), ("down", bc.xr_act, bc.mlp)):
            jobs.append((w[nm], xr, y[:B]))
    nbytes = sum(wt.nbytes + B * wt.K * 2 + B * wt.N * 2 for wt, _, _ in jobs)
    ws = ops.workspace(1 << 26, model.device)

    def run_all():
        st = torch.cuda.current_stream().cuda_stream
        for wt, xr, y in jobs:   # the entry point the step itself uses: activations already in the kernel's input layout
            rc = L.vk_w4_gemm_xrec(wt.packed.data_ptr(), xr.data_ptr(), y.data_ptr(), y.stride(0), B, wt.N, wt.K, ws.data_ptr(),
                                   ws.numel(), st)
            assert rc == 0, rc

    run_all()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run_all()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) * 1e-3 / reps
    return len(jobs), nbytes / len(jobs), sec / len(jobs)


def run_ours(a):
    import torch
    import torch.distributed as dist

    from volundr_mlx_b200 import batch as BT, ops, synth
    from volundr_mlx_b200.volundr import Model, SynthParams

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    kw = {}
    if a.layers:
        full = synth.volundr32b_args()
        kw = dict(num_hidden_layers=a.layers, mixer_types=full.mixer_types[: a.layers],
                  engram_layers=[])   # (no Engram table: the reduced model is a small case for profiler captures)
    args = synth.volundr32b_args(**kw)
    params = SynthParams(args, dev, seed=4, bias_mode="free")
    model = Model(args, params, dev, tp_rank=rank, tp_size=world, group=group)
    if a.prefetch_mb:
        from volundr_mlx_b200 import _lib
        _lib.lib().vk_w4_force_plan(0, a.prefetch_mb)
    del params
    torch.cuda.empty_cache()
    ctx = context_lengths()
    steps_total = a.warmup + a.steps + a.warmup + a.steps + 8
    pages_row = (max(ctx) + steps_total) // 64 + 2
    n_pages = sum((c + steps_total) // 64 + 2 for c in ctx)
    bc = model.make_cache(max_rows=B_ROWS, n_pages=n_pages, max_pages_per_row=pages_row, seed=4)
    bc.fill_synthetic(list(range(B_ROWS)), ctx, seed=4)
    B = bc.B

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    rng = np.random.default_rng(4)
    toks0 = torch.from_numpy(rng.integers(0, args.vocab_valid, size=B).astype(np.int32)).to(dev)

    # ---- device-resident loop: greedy ids feed the next step without leaving the GPU
    BT.forward(model, bc, toks0)
    for _ in range(a.warmup):
        BT.forward(model, bc, bc.greedy[:B])
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.nvtx.range_push("vk_timed")  # lets a profiler pick out the timed steps
    e0.record()
    for _ in range(a.steps):
        BT.forward(model, bc, bc.greedy[:B])
    e1.record()
    barrier()
    torch.cuda.nvtx.range_pop()
    ms_dev = max_over_ranks(e0.elapsed_time(e1)) / a.steps
    clocks = sampler.stop() if rank == 0 else None
    ops.check_status()

    # ---- end to end through the batch API: tokens from pinned host memory, greedy ids back to the host, every step
    pin_in = torch.empty(B, dtype=torch.int32).pin_memory()
    pin_out = torch.empty(B, dtype=torch.int32).pin_memory()
    pin_in.copy_(bc.greedy[:B].cpu())
    for _ in range(a.warmup):
        BT.forward(model, bc, pin_in)
        pin_out.copy_(bc.greedy[:B], non_blocking=True)
        torch.cuda.synchronize()
        pin_in.copy_(pin_out)
    barrier()
    e0.record()
    for _ in range(a.steps):
        BT.forward(model, bc, pin_in)                      # H2D copy of the step's tokens inside
        pin_out.copy_(bc.greedy[:B], non_blocking=True)    # D2H read of the step's result
        torch.cuda.synchronize()
        pin_in.copy_(pin_out)
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1)) / a.steps

    # ---- roofline of the dominant kernel and the step's byte accounting
    peak, peak_kind = measured_peaks()
    n_gemm, bytes_per_launch, sec_per_launch = gemm_roofline(model, bc, torch, ops)
    achieved = bytes_per_launch / sec_per_launch / 1e9
    step_bytes = (model.weight_bytes() + bc.state_bytes_per_step()) * world   # every rank streams its own shard
    launches = bc.kernels_per_step  # counted by the library while the step was captured

    def leave():
        # Every rank is past its last collective here. The step's CUDA graphs hold captured NCCL kernels, so they are
        # released before the communicator goes away.
        if world > 1:
            bc.graphs.clear()
            barrier()
            th = threading.Thread(target=dist.destroy_process_group, daemon=True)
            th.start()
            th.join(20.0)
            if th.is_alive():   # a communicator that will not shut down must not keep a finished run from exiting
                sys.stdout.flush()
                os._exit(0)

    if rank != 0:
        leave()
        return
    cpu = cpu_sample(steps=8, warmup=1) if (world == 1 and not a.no_cpu) else None
    line = {
        "metric": METRIC, "value": B * 1e3 / ms_dev, "unit": "tok/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": ms_dev, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"volundr-32b-shaped W4 g64, {args.num_hidden_layers} layers, {B} ragged rows "
                               f"(ctx {min(ctx)}..{max(ctx)}), greedy decode step",
                   "parallelism": f"tp{world}" + ("" if world == 1 else (" exchange in the consuming kernels over peer memory"
                                                                                 if bc.ar is not None else " NCCL all-reduce")), "l2": "inputs larger than L2 (weights >= 18 GB per step)",
                   "bytes_per_step": step_bytes, "hbm_roofline_frac": step_bytes / (ms_dev * 1e-3) / 1e9 / (peak * world),
                   "hbm_roofline_frac_nominal_8TBs": step_bytes / (ms_dev * 1e-3) / 1e9 / (8000.0 * world)},
        "e2e": {"value": B * 1e3 / ms_e2e, "unit": "tok/s", "h2d_bytes_per_step": B * 4, "d2h_bytes_per_step": B * 4},
        "gpu_launches": launches * a.steps,
        "roofline": {"bound": "hbm", "kernel": "w4_gemm_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": bytes_per_launch * NCU_TRAFFIC_RATIO,
                     "traffic_source": "ncu dram read+write of two shapes (44032x5120: 1.03x, 5120x5120: 0.99x the "
                                       "algorithmic bytes), scaled to the average launch",
                     "peak_kind": peak_kind, "launches_per_step": n_gemm,
                     "bytes_per_launch": bytes_per_launch},
        "clocks": clocks,
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)
    leave()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="debug: only the first L layers (the result is then not the metric)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--prefetch-mb", type=int, default=0,
                    help="tuning: L2 prefetch budget of a GEMM launch in MB (0 = off, the library default)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)


if __name__ == "__main__":
    main()
