"""One W4 GEMM shape in isolation: `python -m volundr_mlx_b200.gemm_case --n 44032 --k 5120 --m 16`.

Runs y = x . dequant(W)^T through vk_w4_gemm (the replacement of mx.quantized_matmul at the call sites
volundr.py:185-190, 377-386, 645-648) over several weight copies, so that consecutive launches read different memory
(more than the L2 holds in total), as one CUDA graph with programmatic dependent launch like the decode step, and
prints the time per launch and the algorithmic GB/s (N*K*0.5625 + M*K*2 + M*N*2 bytes). This is the small case that
profiler captures of the kernel use; it is also the quickest check of a new GPU or driver.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops


def make_weight(N: int, K: int, device, seed: int):
    g = torch.Generator(device="cpu").manual_seed(seed)
    w = torch.randint(-2 ** 31, 2 ** 31 - 1, (N, K // 8), dtype=torch.int32, generator=g).to(device)
    s = (torch.randn(N, K // 64, generator=g).abs() * 0.02 / 8).to(torch.bfloat16).to(device)
    b = (torch.randn(N, K // 64, generator=g) * 0.01).to(torch.bfloat16).to(device)
    return ops.w4_repack(w, s, b, 64)


def run(M: int, N: int, K: int, copies: int, launches: int, replays: int, device=None, tile: bool = False):
    device = device or torch.device("cuda", 0)
    wts = [make_weight(N, K, device, 100 + i) for i in range(copies)]
    x = torch.randn(M, K, device=device).to(torch.bfloat16)
    y = torch.empty(M, N, device=device, dtype=torch.bfloat16)
    gemm = ops.w4_gemm_tile if tile else ops.w4_gemm   # (tile: the tcgen05 kernel for many rows)
    s = torch.cuda.Stream(device)
    with torch.cuda.stream(s):
        for i in range(min(copies, 3)):
            gemm(x, wts[i], y)
        torch.cuda.synchronize(device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for i in range(launches):
                gemm(x, wts[i % copies], y)
        g.replay()
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        for _ in range(replays):
            g.replay()
        e1.record(s)
        torch.cuda.synchronize(device)
    ops.check_status(device)
    us = e0.elapsed_time(e1) * 1e3 / (replays * launches)   # per vk_w4_gemm call: x-record kernel + GEMM kernel
    nbytes = N * K * 0.5625 + M * K * 2 + M * N * 2
    return {"M": M, "N": N, "K": K, "kernel": "tcgen05 tile" if tile else "streaming", "us_per_gemm": us,
            "GBps": nbytes / us / 1e3, "TFLOPs": 2.0 * M * N * K / us / 1e6, "bytes": nbytes, "copies": copies}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=16)
    ap.add_argument("--n", type=int, default=44032)
    ap.add_argument("--k", type=int, default=5120)
    ap.add_argument("--copies", type=int, default=0, help="weight copies (default: enough for 400 MB)")
    ap.add_argument("--launches", type=int, default=12)
    ap.add_argument("--replays", type=int, default=5)
    ap.add_argument("--tile", action="store_true", help="use vk_w4_gemm_tile (tcgen05, for many rows)")
    ap.add_argument("--tile-shape", default="0,0", help="force the tile kernel's weight rows per CTA and row tiles per CTA")
    a = ap.parse_args()
    if a.tile:
        from . import _lib
        tn, ml = (int(v) for v in a.tile_shape.split(","))
        _lib.check(_lib.lib().vk_w4_tile_force(tn, ml), "vk_w4_tile_force")
    import os
    if os.environ.get("VK_W4_SELECT"):   # 0: mma.sync kernel, 2 / 3: the tcgen05 kernel with that expansion-to-accumulation lag
        from . import _lib
        _lib.lib().vk_w4_select(int(os.environ["VK_W4_SELECT"]))
    copies = a.copies or max(2, int(400e6 // (a.n * a.k * 0.5625)) + 1)
    print(json.dumps(run(a.m, a.n, a.k, copies, a.launches, a.replays, tile=a.tile)))


if __name__ == "__main__":
    main()
