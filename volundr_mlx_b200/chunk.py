"""T tokens per row through every layer in one pass over the weights: the tile the reference reaches through
batch_spec.verify_forward (batch_spec.py:107-158: B x T verify) and, with one row, through the prefill chunks of
session.prefill_iter (session.py:351-387) / verify.forward_iter (spec/verify.py:180-226).

The tokens run as R "virtual rows", the requests' rows one after another: row off[b] + t is token t of request b, at
position pos[b] + t, on the page table of request b. Requests may bring different numbers of tokens (ragged chunks:
R = the sum of the counts, nothing is padded); with T tokens each, off[b] = b * T. Linears see all R rows at once (vk_w4_gemm: wide passes; vk_bf16_gemm_packed), the row-wise
kernels (mHC, norms, SiLU, Engram) are the decode step's kernels on R rows, attention is the decode attention with R
query rows (each sees the keys up to its own position: all rows' K/V are written before anything is attended, blocks
that close inside the window are pooled in a second pass), the KDA recurrence is vk_kda_chunk. Nothing here waits for
a per-token step of another layer.

forward_chunk(..., write=False) is the verify pass: K/V of all T tokens go into the pages (positions a commit does not
keep are simply never reached), the KDA state and the Engram window stay as they were, and what a commit needs
(the KDA layers' inputs) is kept. commit_chunk(accepted) replays the KDA recurrence over the accepted prefix of every
row (vk_kda_chunk with `accept`), moves the Engram window, returns pages opened for rejected positions and advances
the positions. forward_chunk(..., write=True) commits all T tokens at once (a prefill chunk).
Tensor parallel: the shards' partial products of out_proj / o_proj and down_proj ([R, hidden] bf16, megabytes at
R in the hundreds) are summed with NCCL all-reduces between the kernels (bandwidth-bound at this size, unlike the
decode step's 160 KB exchanges, which live inside the consuming kernels); logits come back as the rank's vocabulary
shard, greedy tokens from per-rank (max, index) pairs, all-gathered and merged.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib, ops
from . import batch as BT

BF16 = torch.bfloat16
PAGE = BT.PAGE
_p = BT._p


class ChunkScratch:
    """Activations of up to R virtual rows (capacities are powers of two, so a cache meets only a few of them)."""

    def __init__(self, model, bc, R):
        a, d, D = model.args, model.device, model.args.hidden_size
        bf = dict(dtype=BF16, device=d)
        f32 = dict(dtype=torch.float32, device=d)
        i32 = dict(dtype=torch.int32, device=d)
        self.R = R
        wid = max(w["proj"].N for w in model.layers)
        self.H = torch.zeros((R, 4, D), **bf)
        self.hn, self.x_in, self.h = (torch.zeros((R, D), **bf) for _ in range(3))
        self.post, self.res, self.dyn = torch.zeros((R, 4), **f32), torch.zeros((R, 16), **f32), torch.zeros((R, 24), **f32)
        self.proj = torch.zeros((R, wid), **bf)
        self.mix = torch.zeros((R, max(model.HV * 128, model.Hq * 128)), **bf)
        self.r, self.h2, self.hn2, self.mlp = (torch.zeros((R, D), **bf) for _ in range(4))
        self.gu = torch.zeros((R, 2 * model.I), **bf)
        self.act = torch.zeros((R, model.I), **bf)
        self.logits = torch.zeros((R, model.vocab_shard), **bf)
        self.greedy = torch.zeros(R, **i32)
        self.pairs = torch.zeros((R, 2), **i32)
        self.pairs_all = torch.zeros((model.tp_size, R, 2), **i32)
        self.tok = torch.zeros(R, **i32)
        self.pos = torch.zeros(R, **i32)
        self.table = torch.full((R, bc.max_pages), -1, **i32)
        self.row_map = torch.zeros(R, **i32)
        self.engram_prev = torch.full((R, max(bc.keep, 1)), -1, **i32)
        self.engram_rows = torch.zeros((R, max(len(a.engram_orders), 1)), **i32)
        self.q = torch.zeros((R, model.Hq, 128), **bf)
        if bc.indexer:
            self.qi = torch.zeros((R, a.bcsa_index_heads, a.bcsa_index_dim), **bf)
            self.idxq = torch.zeros((R, a.bcsa_index_heads * a.bcsa_index_dim), **bf)
            self.idxk = torch.zeros((R, a.bcsa_index_dim), **bf)
            self.ikc = torch.zeros((R, a.bcsa_index_dim), **bf)     # normed indexer key of every virtual row
            self.first_pos = torch.zeros(R, **i32)                  # where the chunk began for the row's request
        self.sel = torch.full((R, max(bc.NS, 1), max(a.bcsa_topk, 1)), -1, **i32)
        self.nsel = torch.zeros((R, max(bc.NS, 1)), **i32)
        self.sel_scratch = torch.zeros((R, max(bc.NS, 1), bc.max_blocks), **i32)
        self.part = torch.zeros((R, model.Hq, max(bc.nsplit_bcsa, bc.nsplit_dense), 130), **f32)
        if a.engram_layers:
            self.eng_e = torch.zeros((R, a.engram_dim * len(a.engram_orders)), **bf)
            self.eng_val = torch.zeros((R, D), **bf)


class ChunkHandle:
    """What a verify pass leaves for its commit (the reference's `rec`, batch_spec.py:128): the rows' token counts and
    start positions, the Engram id window, the KDA layers' inputs (the commit replays the recurrence over the accepted
    prefix), the chunk's indexer keys per BCSA layer (the commit stores the open block's), plus the pass's outputs."""

    def __init__(self, model, lens, pos0, window, kda_inputs, off, ik):
        self.model = model
        self.lens, self.pos0, self.window, self.kda_inputs, self.off, self.ik = lens, pos0, window, kda_inputs, off, ik
        self.offs = [sum(lens[:b]) for b in range(len(lens))]      # the requests' first virtual rows, on the host
        self.T = max(lens)
        self.greedy = None
        self.features = None


def _get_scratch(model, bc, R):
    """Scratch for R rows: the smallest power-of-two capacity that holds them, the last few capacities kept. It lives
    on the cache object, so it can never outlive the shapes it was made for."""
    cap = scratch_capacity(R)
    held = bc.__dict__.setdefault("_chunk_scratch", {})
    if cap in held:
        held[cap] = held.pop(cap)                    # most recently used last
    else:
        while len(held) >= 4:
            held.pop(next(iter(held)))
        held[cap] = ChunkScratch(model, bc, cap)
    return held[cap]


def virtual_rows(lens, device=None):
    """The layout of a chunk's virtual rows: request b brings lens[b] tokens and owns the rows off[b] .. off[b] +
    lens[b] - 1. Returns (off [B] int32, rows [R] long: the request of every virtual row, tpos [R] long: its token
    index within the request)."""
    lens_t = torch.tensor(list(lens), dtype=torch.long, device=device)
    off = torch.cumsum(lens_t, 0) - lens_t
    rows = torch.arange(len(lens), device=device).repeat_interleave(lens_t)
    tpos = torch.arange(int(lens_t.sum()), device=device) - off[rows]
    return off.to(torch.int32), rows, tpos


def scratch_capacity(R: int) -> int:
    """Rows of the scratch that serves a chunk of R virtual rows: the next power of two, at least 16."""
    cap = 16
    while cap < R:
        cap *= 2
    return cap


def _open_pages(bc, lens, lens_t):
    """Pages for the positions pos .. pos + lens[b] - 1 of every row, handed out on the GPU (vk_pages_open); the host
    only checks the rows' page tables for room. An exhausted pool shows in the device status word."""
    for b, p0 in enumerate(bc._pos):
        assert (p0 + lens[b] + PAGE - 1) // PAGE <= bc.max_pages, "row would outgrow its page table"
    _lib.check(_lib.lib().vk_pages_open(_p(bc.pos), _p(lens_t), _p(bc.table), bc.max_pages, _p(bc.free_list), _p(bc.free_top),
                                        bc.B, torch.cuda.current_stream().cuda_stream), "vk_pages_open")


def _store_open_keys(bc, lst, ikc, off, pos0, kept):
    """off: the requests' first virtual rows (host ints). The open block's indexer keys after request b kept kept[b] tokens of a chunk that began at pos0[b]: the ring
    IK [row, C, Di] gets the keys of the positions of the last, unfinished block that the chunk brought (those in front
    of the chunk are in the ring already; BCSACache.update, volundr.py:526-533; batch_spec.py:151-158)."""
    C = bc.args.bcsa_compress
    rows, slots, src = [], [], []
    for b, (p0, n) in enumerate(zip(pos0, kept)):
        end = p0 + n
        for t in range(max(end - end % C, p0), end):
            rows.append(b)
            slots.append(t % C)
            src.append(off[b] + t - p0)
    if rows:
        dev = ikc.device
        ix = lambda v: torch.tensor(v, dtype=torch.long, device=dev)
        lst["IK"][ix(rows), ix(slots)] = ikc[ix(src)]


def forward_chunk(model, bc, toks, write=False, logits_at=None, capture=()):
    """toks [B][T], or one list of tokens per row with different lengths (a ragged chunk). Returns (logits, greedy,
    handle): logits [B, T, V] bf16 and greedy [B, T] int32 for T tokens per row; for a ragged chunk the LM head runs on
    one token per row (logits_at, default each row's last), logits [B, 1, V], greedy [B, 1]. write=False: a verify
    pass, to be followed by commit_chunk(model, bc, handle, accepted); write=True: all tokens are committed (handle is
    None). logits_at [B] (token index per row) restricts the LM head to that token of every row (what feeding a prompt
    needs: the logits after its last token). capture: layer indices whose entry stream-0 residual is kept
    (batch.py:540-541; batch_spec.py:121-122): handle.features [B, T, len(capture) * hidden] ([R, ...] for a ragged
    chunk), also returned by the generator form."""
    gen = forward_chunk_iter(model, bc, toks, write=write, logits_at=logits_at, capture=capture)
    try:
        while True:
            next(gen)
    except StopIteration as e:
        return e.value


def forward_chunk_iter(model, bc, toks, write=False, logits_at=None, capture=(), yield_layers=True):
    """forward_chunk as a generator: yields ("layer", i) after the kernels of layer i have been enqueued, so that a
    scheduler can stop feeding a long chunk when its time slice is spent and run decode steps of other caches in between
    (session.prefill_iter with yield_layers, session.py:351-387; verify.forward_iter, spec/verify.py:180-226). The
    cache `bc` itself must not be stepped before the generator has finished. Returns forward_chunk's value."""
    L = _lib.lib()
    tp = model.tp_size > 1
    a, D = model.args, model.args.hidden_size
    dev = bc.pos.device
    if torch.is_tensor(toks):
        toks = toks.tolist()
    toks = [[int(x) for x in row] for row in toks]
    lens = [len(row) for row in toks]
    B, T, R = len(toks), max(lens), sum(lens)
    assert B == bc.B and min(lens) >= 1
    ragged = min(lens) != T
    if ragged and logits_at is None:
        logits_at = [n - 1 for n in lens]
    t_in = torch.tensor([row + [0] * (T - len(row)) for row in toks], dtype=torch.int32).to(dev)   # [B, T], padded
    s = _get_scratch(model, bc, R)
    BT.model_warm(model)
    acc_all = torch.tensor(lens, dtype=torch.int32, device=dev)
    _open_pages(bc, lens, acc_all)
    st = torch.cuda.current_stream().cuda_stream
    eps = a.rms_norm_eps
    ck = _lib.check
    # ---- virtual rows: request and token index of each
    off_t, rows, tpos = virtual_rows(lens, dev)
    s.row_map[:R].copy_(rows.to(torch.int32))
    s.tok[:R].copy_(t_in[rows, tpos])
    s.pos[:R].copy_(bc.pos[:B][rows] + tpos.to(torch.int32))
    s.table[:R].copy_(bc.table[:B][rows])
    if bc.indexer:
        s.first_pos[:R].copy_(bc.pos[:B][rows])
    window = None
    if a.engram_layers and bc.keep > 0:
        window = torch.cat([bc.engram_prev[:B, : bc.keep], t_in], dim=1)          # [B, keep + T]
        s.engram_prev[:R].copy_(window.unfold(1, bc.keep, 1)[rows, tpos])
    ws = ops.workspace(max(1 << 26, L.vk_w4_workspace_bytes(R, max(w["gate_up"].N for w in model.layers), D)), dev)

    tile_ws = None
    if R >= 64:
        kmax = max(max(w[nm].K for nm in ("proj", "out", "gate_up", "down")) for w in model.layers)
        nmax = max(max(w[nm].N for nm in ("proj", "out", "gate_up", "down")) for w in model.layers)
        need = max(L.vk_w4_tile_workspace_bytes_n(R, w[nm].N, w[nm].K) for w in model.layers for nm in ("proj", "out", "gate_up", "down"))
        tile_ws = ops.tile_workspace(max(need, L.vk_w4_tile_workspace_bytes(R, kmax)), dev)   # (zeroed once: its head holds counters)
        del nmax

    def gemm(x, wt, y):
        # 64 rows and more: the tcgen05 tile kernel; fewer: the streaming kernel's passes
        if R >= 64:
            ck(L.vk_w4_gemm_tile(_p(wt.packed), _p(x), x.stride(0), _p(y), y.stride(0), R, wt.N, wt.K, _p(tile_ws),
                                 tile_ws.numel(), st), "vk_w4_gemm_tile")
        else:
            ck(L.vk_w4_gemm(_p(wt.packed), _p(x), x.stride(0), _p(y), y.stride(0), R, wt.N, wt.K, _p(ws), ws.numel(), st),
               "vk_w4_gemm")

    def allreduce(t):
        if tp:
            torch.distributed.all_reduce(t, group=model.group)

    w0 = model.layers[0]
    ck(L.vk_embed(_p(s.tok), _p(model.embed), _p(w0["mhc_norm"]), _p(s.H), _p(s.hn),
                  _p(s.engram_prev) if a.engram_layers else None, _p(s.engram_rows), bc.orders,
                  len(a.engram_orders) if a.engram_layers else 0, a.engram_rows, R, D, eps, st), "vk_embed")
    kda_inputs, ik_kept, caps = [], {}, []
    nl = len(model.layers)
    # tiles of up to 16 consecutive rows of one request for the attention kernel that reads a tile's keys once
    offs = [sum(lens[:b]) for b in range(B)]
    tiles = [(offs[b] + t0, min(16, lens[b] - t0)) for b in range(B) for t0 in range(0, lens[b], 16)]
    tile_t = torch.tensor(tiles, dtype=torch.int32).t().contiguous().to(dev)          # [2, tiles]
    use_tiles = bc.tile_attention and T > 1
    for i, (w, lst) in enumerate(zip(model.layers, bc.layers)):
        if i in capture:
            caps.append(s.H[:R, 0].clone())
        ck(L.vk_mhc_mix_norm(_p(s.H), _p(s.hn), _p(w["dyn"]), _p(w["pre_s"]), _p(w["post_s"]), _p(w["res_s"]), _p(w["ln_in"]),
                             _p(s.x_in), _p(s.h), None, _p(s.post), _p(s.res), _p(s.dyn), R, D, a.mhc_sinkhorn_iters, eps, st),
           "vk_mhc_mix_norm")
        gemm(s.h, w["proj"], s.proj)
        if w["mixer"] == "kda":
            nmix = model.HV * 128
            if not write:
                kda_inputs.append((i, s.proj[:R, : w["proj"].N].clone(), s.h[:R].clone()))
            ck(L.vk_kda_chunk_ragged(_p(s.proj), s.proj.stride(0), w["off_z"], w["off_fd"], _p(s.h), _p(w["in_proj_b"]),
                                     _p(w["f_up"]), _p(w["conv_w"]), _p(w["A_log"]), _p(w["dt_bias"]), _p(w["gnorm"]),
                                     _p(lst["conv"]), _p(bc.parity), lst["conv"][0].numel(), _p(lst["S"]), _p(s.mix),
                                     _p(acc_all), _p(off_t), 1 if write else 0, B, T, D, model.Hk, model.HV, 128, 128,
                                     a.kda_gate_rank, eps, st), "vk_kda_chunk_ragged")
        else:
            bcsa = w["mixer"] == "bcsa"
            g = bc.geom[w["mixer"]]
            nmix = model.Hq * 128
            idx = bcsa and bc.indexer
            if idx:
                ck(L.vk_bf16_gemm(_p(s.h), D, _p(w["idx_q"]), None, _p(s.idxq), s.idxq.stride(0), R, w["idx_q"].shape[0], D, st),
                   "vk_bf16_gemm")
                ck(L.vk_bf16_gemm(_p(s.h), D, _p(w["idx_k"]), None, _p(s.idxk), s.idxk.stride(0), R, w["idx_k"].shape[0], D, st),
                   "vk_bf16_gemm")
            for mode in (1, 2):   # write every row's K / V first, pool the blocks that close afterwards
                ck(L.vk_attn_prep_chunk(ctypes.byref(g), _p(s.proj), s.proj.stride(0), w["off_k"], w["off_v"],
                                        _p(s.idxq) if idx else None, _p(s.idxk) if idx else None, _p(w["q_norm"]),
                                        _p(w["k_norm"]), _p(w["idx_norm"]) if idx else None, _p(s.pos), _p(s.table), _p(s.q),
                                        _p(s.qi) if idx else None, _p(lst["K"]), _p(lst["V"]), _p(lst.get("PK")),
                                        _p(lst.get("PV")), _p(lst.get("BK")), _p(lst.get("IK")), R, model.rope_dims,
                                        float(a.rope_theta), eps, mode, _p(s.row_map), _p(s.ikc) if idx else None,
                                        _p(s.first_pos) if idx else None, st), "vk_attn_prep_chunk")
                if not bcsa:
                    break   # (a dense layer pools nothing)
            if idx:   # the open block's indexer keys: now for a chunk that is committed as it is, else at the commit
                if write:
                    _store_open_keys(bc, lst, s.ikc, offs, bc._pos, lens)
                else:
                    ik_kept[i] = s.ikc[:R].clone()
            if bcsa:
                ck(L.vk_bcsa_select(ctypes.byref(g), _p(s.qi) if idx else _p(s.q), _p(lst["BK"]) if idx else _p(lst["PK"]),
                                    _p(s.pos), _p(s.table), _p(s.sel_scratch), bc.max_blocks, _p(s.sel), _p(s.nsel), R, st),
                   "vk_bcsa_select")
            done = False
            if use_tiles:
                W, C = (a.bcsa_window, a.bcsa_compress) if bcsa else (0, 1)
                nv_cap = max(max(0, (p0 + n - W) // C) for p0, n in zip(bc._pos, lens)) if bcsa else 0
                nsplit = max(1, min(16, -(-4 * 148 // (len(tiles) * model.KVH))))
                rc = L.vk_attend_chunk(ctypes.byref(g), _p(s.q), _p(lst["K"]), _p(lst["V"]), _p(lst.get("PK")), _p(lst.get("PV")),
                                       _p(s.pos), _p(s.table), _p(s.sel), _p(s.nsel), _p(tile_t[0]), _p(tile_t[1]), len(tiles),
                                       nv_cap, _p(s.proj), s.proj.stride(0), _p(s.part), nsplit, _p(s.mix), R, st)
                if rc != -3:       # (-3: the union's bookkeeping does not fit shared memory: one query row at a time)
                    ck(rc, "vk_attend_chunk")
                    done = True
            if not done:
                ck(L.vk_attend_decode(ctypes.byref(g), _p(s.q), _p(lst["K"]), _p(lst["V"]), _p(lst.get("PK")), _p(lst.get("PV")),
                                      _p(s.pos), _p(s.table), _p(s.sel), _p(s.nsel), _p(s.proj), s.proj.stride(0), _p(s.part),
                                      bc.nsplit_bcsa if bcsa else bc.nsplit_dense, _p(s.mix), None, R, st), "vk_attend_decode")
        gemm(s.mix[:, :nmix], w["out"], s.r)
        allreduce(s.r[:R])
        ck(L.vk_add_rmsnorm(_p(s.x_in), _p(s.r), _p(w["ln_post"]), _p(s.h2), _p(s.hn2), None, R, D, eps, 1, st), "vk_add_rmsnorm")
        gemm(s.hn2, w["gate_up"], s.gu)
        ck(L.vk_silu_mul(_p(s.gu), _p(s.act), None, R, model.I, s.gu.stride(0), st), "vk_silu_mul")
        gemm(s.act, w["down"], s.mlp)
        allreduce(s.mlp[:R])
        eng = "eng_norm" in w
        val = None
        if eng:
            ptrs, lds, c0 = w["eng_ptrs"]
            ck(L.vk_engram_gather(ptrs.ctypes.data_as(ctypes.c_void_p), lds.ctypes.data_as(ctypes.c_void_p),
                                  c0.ctypes.data_as(ctypes.c_void_p), _p(s.engram_rows), _p(w["eng_norm"]), _p(s.eng_e), R,
                                  len(a.engram_orders), a.engram_dim, eps, st), "vk_engram_gather")
            val = s.eng_e
            if a.engram_value:
                ck(L.vk_bf16_gemm(_p(s.eng_e), s.eng_e.stride(0), _p(w["eng_value"]), None, _p(s.eng_val), D, R, D,
                                  s.eng_e.shape[1], st), "vk_bf16_gemm")
                val = s.eng_val
        last = i + 1 == nl
        w_next = model.norm_w if last else model.layers[i + 1]["mhc_norm"]
        ck(L.vk_mhc_combine_norm(_p(s.H), _p(s.h2), _p(s.mlp), _p(s.x_in), _p(s.post), _p(s.res), _p(w_next), _p(s.hn),
                                 _p(val) if eng else None, _p(w["eng_gate_w"]) if eng else None,
                                 _p(w["eng_gate_b"]) if eng else None, None, R, D, 1 if last else 0, eps, st),
           "vk_mhc_combine_norm")
        if yield_layers and not last:
            yield ("layer", i)
    V = model.vocab_shard
    hn, RL, TL = s.hn, R, T            # rows that go through the LM head
    if logits_at is not None:
        at = torch.as_tensor(logits_at, dtype=torch.long).to(dev)
        assert at.shape == (B,)
        assert all(0 <= int(x) < lens[b] for b, x in enumerate(logits_at))
        hn = s.hn.index_select(0, off_t.long() + at)
        RL, TL = B, 1
    if isinstance(model.lm_head, ops.BF16Weight):
        ck(L.vk_bf16_gemm_packed(_p(model.lm_head.packed), _p(hn), D, _p(s.logits), s.logits.stride(0), RL, V, D, _p(ws),
                                 ws.numel(), st), "vk_bf16_gemm_packed")
    else:
        ck(L.vk_bf16_gemm(_p(hn), D, _p(model.lm_head), None, _p(s.logits), s.logits.stride(0), RL, V, D, st), "vk_bf16_gemm")
    if not tp:
        ck(L.vk_argmax(_p(s.logits), s.logits.stride(0), min(a.vocab_valid, V), _p(s.greedy), RL, st), "vk_argmax")
    else:
        ck(L.vk_argmax_pairs(_p(s.logits), s.logits.stride(0), max(0, min(a.vocab_valid - model.vocab0, V)), model.vocab0,
                             _p(s.pairs), RL, st), "vk_argmax_pairs")
        gathered = s.pairs_all.view(-1)[: model.tp_size * RL * 2].view(model.tp_size, RL, 2)
        torch.distributed.all_gather_into_tensor(gathered, s.pairs[:RL], group=model.group)
        ck(L.vk_argmax_merge(_p(s.pairs_all), model.tp_size, _p(s.greedy), RL, st), "vk_argmax_merge")
    logits = s.logits[:RL].view(B, TL, V)
    greedy = s.greedy[:RL].view(B, TL)
    handle = ChunkHandle(model, lens, list(bc._pos), window, kda_inputs, off_t, ik_kept)
    handle.greedy = greedy
    if caps:
        f = torch.cat(caps, dim=-1)
        handle.features = f if ragged else f.view(B, T, -1)
    if write:
        _finish(model, bc, handle, lens, replay=False)
        handle.kda_inputs, handle.ik = [], {}      # (nothing left to commit; the outputs stay readable)
        return logits, greedy, (handle if capture else None)
    return logits, greedy, handle


def _finish(model, bc, h: ChunkHandle, acc, replay):
    L = _lib.lib()
    a, D = model.args, model.args.hidden_size
    B, T = bc.B, h.T
    R = sum(h.lens)
    dev = bc.pos.device
    st = torch.cuda.current_stream().cuda_stream
    has_kda = any("S" in lst for lst in bc.layers)
    if replay and has_kda:
        acc_t = torch.tensor(acc, dtype=torch.int32, device=dev)
        scratch_out = torch.empty((R, model.HV * 128), dtype=BF16, device=dev)
        for i, proj, hin in h.kda_inputs:
            w, lst = model.layers[i], bc.layers[i]
            _lib.check(L.vk_kda_chunk_ragged(_p(proj), proj.stride(0), w["off_z"], w["off_fd"], _p(hin), _p(w["in_proj_b"]),
                                             _p(w["f_up"]), _p(w["conv_w"]), _p(w["A_log"]), _p(w["dt_bias"]),
                                             _p(w["gnorm"]), _p(lst["conv"]), _p(bc.parity), lst["conv"][0].numel(),
                                             _p(lst["S"]), _p(scratch_out), _p(acc_t), _p(h.off), 1, B, T, D, model.Hk,
                                             model.HV, 128, 128, a.kda_gate_rank, a.rms_norm_eps, st),
                       "vk_kda_chunk_ragged")
    if replay:
        for i, ikc in h.ik.items():
            _store_open_keys(bc, bc.layers[i], ikc, h.offs, h.pos0, acc)
    if has_kda:          # the conv windows now sit in the other buffer, as after a decode step
        bc.parity ^= 1
        bc.steps += 1
    if h.window is not None:
        idx = torch.tensor(acc, dtype=torch.long, device=dev).unsqueeze(1) + torch.arange(bc.keep, device=dev).unsqueeze(0)
        bc.engram_prev[:B, : bc.keep] = torch.gather(h.window, 1, idx)
    # pages opened for positions the rows do not keep go back to the pool (on the GPU: no host round trip)
    pages = lambda n: (n + PAGE - 1) // PAGE
    back = [(b, pages(h.pos0[b] + acc[b]), pages(h.pos0[b] + h.lens[b])) for b in range(B)]
    back = [x for x in back if x[2] > x[1]]
    if back:
        bc.release_pages(back, reverse=False)
    bc._pos = [h.pos0[b] + acc[b] for b in range(B)]
    bc.pos[:B] = torch.tensor(bc._pos, dtype=torch.int32, device=dev)


def commit_chunk(model, bc, handle: ChunkHandle, accepted):
    """accepted[b] in 0..T: the number of tokens of the verify pass request b keeps (batch_spec.commit,
    batch_spec.py:160-199)."""
    acc = [int(x) for x in accepted]
    assert len(acc) == bc.B and all(0 <= n <= handle.lens[b] for b, n in enumerate(acc))
    _finish(model, bc, handle, acc, replay=True)
