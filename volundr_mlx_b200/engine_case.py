"""The continuous-batching workload on the synthetic 32B-shaped model, end to end through engine.BatchEngine:
`python -m volundr_mlx_b200.engine_case --requests 16 --new 64 --prefill-chunk 128`.

Sixteen requests with prompts log-uniform in 256..20K tokens (the reference's batched workload: scheduler.py:72-560
driven by worker.py), greedy decoding of `--new` tokens each; prompts are fed in ragged chunks of up to
`--prefill-chunk` tokens per row (0: one token per step). Prints one JSON line: wall time, prompt and generated
tokens per second, the number of chunk steps and decode steps. Synthetic weights, seeded.
"""
from __future__ import annotations

import argparse
import json
import time

import numpy as np
import torch

from . import ops, synth
from .engine import BatchEngine
from .volundr import Model, SynthParams


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=16)
    ap.add_argument("--rows", type=int, default=16)
    ap.add_argument("--new", type=int, default=64)
    ap.add_argument("--lo", type=int, default=256)
    ap.add_argument("--hi", type=int, default=20000)
    ap.add_argument("--prefill-chunk", type=int, default=128)
    ap.add_argument("--layers", type=int, default=0, help="0 = all 72")
    ap.add_argument("--slice-ms", type=float, default=0.0,
                    help="> 0: prompts are prefilled on a cache of their own in time slices of this many ms between decode steps")
    ap.add_argument("--warm-graphs", action="store_true", help="capture the step's graph for every batch size before the clock starts")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    kw = {}
    if a.layers:
        full = synth.volundr32b_args()
        kw = dict(num_hidden_layers=a.layers, mixer_types=full.mixer_types[: a.layers], engram_layers=[])
    args = synth.volundr32b_args(**kw)
    model = Model(args, SynthParams(args, dev, seed=4, bias_mode="free"), dev)
    torch.cuda.empty_cache()
    rng = np.random.default_rng(4)
    lens = np.exp(rng.uniform(np.log(a.lo), np.log(a.hi), size=a.requests)).astype(int)
    pages_row = (int(lens.max()) + a.new) // 64 + 2
    eng = BatchEngine(model, max_rows=a.rows, n_pages=int(sum((n + a.new) // 64 + 2 for n in lens)) + 8,
                      max_pages_per_row=pages_row, prefill_chunk=a.prefill_chunk, slice_ms=a.slice_ms)
    if a.warm_graphs:
        eng.warm_graphs()
    for n in lens:
        eng.submit(rng.integers(0, args.vocab_valid, size=int(n)).tolist(), a.new)
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    steps = 0
    while eng.waiting or eng.running or eng.prefilling:
        eng.step()
        steps += 1
        if all(r.done for r in eng.running.values()) and not eng.waiting and not eng.prefilling:
            break
    torch.cuda.synchronize(dev)
    wall = time.perf_counter() - t0
    ops.check_status(dev)
    n_prompt, n_new = int(lens.sum()), a.requests * a.new
    print(json.dumps({"requests": a.requests, "prompt_tokens": n_prompt, "new_tokens": n_new, "wall_s": wall,
                      "tokens_per_s": (n_prompt + n_new) / wall, "steps": steps, "chunk_steps": eng.chunk_steps,
                      "prefill_chunk": a.prefill_chunk, "layers": len(model.layers), "slice_ms": a.slice_ms,
                      "slices": eng.stats["slices"], "longest_gap_between_decode_steps_s": eng.stats["stall_s_max"]}))


if __name__ == "__main__":
    main()
