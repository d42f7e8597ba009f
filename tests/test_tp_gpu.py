"""Tensor-parallel decode on 2 GPUs (NCCL) against the single-GPU run of the same model: same greedy tokens, logits
of each vocabulary shard within bf16 tolerance. Skipped on a box with fewer than 2 GPUs."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out, fused):
    import torch.distributed as dist

    from volundr_mlx_b200 import batch as BT, ops, synth
    from volundr_mlx_b200.volundr import Model

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", VK_TP_FUSED=fused)
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        args = synth.small_args()
        params = synth.make_params(args, seed=9)
        tp = Model(args, params, dev, tp_rank=rank, tp_size=world, group=dist.group.WORLD)
        bc = tp.make_cache(max_rows=4, n_pages=32, max_pages_per_row=4)
        assert (bc.ar is not None) == (fused == "1")
        bc.apply(join=["a", "b", "c"])
        ref = Model(args, params, dev)
        bc1 = ref.make_cache(max_rows=4, n_pages=32, max_pages_per_row=4)
        bc1.apply(join=["a", "b", "c"])
        rng = np.random.default_rng(0)
        worst, merged_ok, agree, clear = 0.0, 0, 0, 0
        v0 = tp.vocab0
        for t in range(30):
            toks = rng.integers(0, args.vocab_valid, size=3).tolist()
            lg, _ = BT.forward(tp, bc, toks)
            l1, _ = BT.forward(ref, bc1, toks)
            a, b = lg.float(), l1.float()[:, v0:v0 + lg.shape[1]]
            worst = max(worst, float((a - b).abs().max() / l1.float().abs().max()))
            # the merged greedy token is the first maximum of the ranks' shards put side by side
            shards = [torch.empty_like(lg) for _ in range(world)]
            dist.all_gather(shards, lg.contiguous())
            full = torch.cat(shards, dim=1)[:, :args.vocab_valid].float()
            merged_ok += int(torch.equal(bc.greedy[:3].long(), full.argmax(dim=1)))
            # against the single-GPU run the token may differ only where its two best logits are a near-tie
            top2 = l1.float()[:, :args.vocab_valid].topk(2, dim=1).values
            gap = (top2[:, 0] - top2[:, 1]) / l1.float().abs().max()
            for r in range(3):
                if float(gap[r]) > 4e-2:
                    clear += 1
                    agree += int(int(bc.greedy[r]) == int(bc1.greedy[r]))
        # the chunk path under tensor parallelism: 3 rows x 24 tokens (72 virtual rows: the tcgen05 tile GEMM on the
        # shards, NCCL all-reduces of [72, hidden]) against the single-GPU chunk, then decode goes on from its state
        from volundr_mlx_b200 import chunk as CH

        toks = rng.integers(0, args.vocab_valid, size=(3, 24)).tolist()
        lg, gr, _ = CH.forward_chunk(tp, bc, toks, write=True)
        l1, g1, _ = CH.forward_chunk(ref, bc1, toks, write=True)
        a, b = lg.float(), l1.float()[:, :, v0:v0 + lg.shape[2]]
        worst = max(worst, float((a - b).abs().max() / l1.float().abs().max()))
        shards = [torch.empty_like(lg) for _ in range(world)]
        dist.all_gather(shards, lg.contiguous())
        full = torch.cat(shards, dim=2)[:, :, :args.vocab_valid].float()
        chunk_ok = int(torch.equal(gr.long(), full.argmax(dim=2)))
        for t in range(4):
            toks = rng.integers(0, args.vocab_valid, size=3).tolist()
            lg, _ = BT.forward(tp, bc, toks)
            l1, _ = BT.forward(ref, bc1, toks)
            a, b = lg.float(), l1.float()[:, v0:v0 + lg.shape[1]]
            worst = max(worst, float((a - b).abs().max() / l1.float().abs().max()))
        merged_ok += chunk_ok - 1          # (30 stays the expected count when the chunk's merged tokens are right)
        ops.check_status()
        out.put((rank, worst, merged_ok, agree, clear))
        out.close()
        out.join_thread()
        # captured graphs hold NCCL kernels: release them before the communicator, and never let a communicator that
        # will not shut down keep a finished worker alive
        bc.graphs.clear()
        bc1.graphs.clear()
        torch.cuda.synchronize()
        dist.barrier()
    finally:
        import threading

        th = threading.Thread(target=dist.destroy_process_group, daemon=True)
        th.start()
        th.join(20.0)
        if th.is_alive():
            os._exit(0)


@pytest.mark.parametrize("fused", ["1", "0"], ids=["peer-exchange", "nccl"])
def test_tp2_matches_single_gpu(fused):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out, fused)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        res = [out.get(timeout=240) for _ in procs]
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    finally:
        for p in procs:
            if p.is_alive():
                p.kill()
    for rank, worst, merged_ok, agree, clear in res:
        assert worst < 3e-2, (rank, worst)       # different summation split of the row-parallel products
        assert merged_ok == 30, (rank, merged_ok)
        assert agree == clear, (rank, agree, clear)
