"""Batched decode with per-row positions: B live sequences of different lengths, one token each per step.

Mirrors the reference's batch.py: `BatchCache(model)` (batch.py:323-515: `.B .pos .keys .row(key) .apply(leave, join)
.capture_row`) and `forward(model, bc, toks, capture) -> (logits [B, V], features)` (batch.py:518-554). Differences
that come with the hardware:
  * Rows live in fixed slots 0..B-1 of preallocated device buffers; positions, the page table and the page free
    list live on the GPU and advance there, so a step launches the same kernels with the same arguments every time
    and is replayed as one CUDA graph (the reference rebuilds a lazy graph per step and pipelines the host work,
    batch.py:368-414; here there is no per-step host work to hide).
  * Attention K/V live in 64-token pages of a shared pool instead of per-row rings padded to the longest row
    (batch.py:8-15); BCSAStep's host-side index lists (batch.py:94-122) are computed inside the kernels.
  * Snapshots are clones (`capture_row`): PyTorch has no copy-on-write arrays (session.py:13-28 relies on MLX's).
"""
import ctypes
import math
import os

import numpy as np
import torch

from . import _lib, ops
from . import session as SS
from .volundr import BF16, Model

PAGE = 64


def _p(t):
    return None if t is None else t.data_ptr()


class _Geom(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in ("Hq", "KVH", "D", "W", "C", "topk", "IH", "Di", "NS", "far_tokens",
                                            "max_pages", "n_pages")]


class BatchCache:
    def __init__(self, model: Model, max_rows: int = 16, n_pages: int = 1024, max_pages_per_row: int = None, seed: int = 0):
        a, d = model.args, model.device
        self.model, self.args, self.S = model, a, max_rows
        self.keys, self._pos = [], []
        self.n_pages = n_pages
        self.max_pages = max_pages_per_row or n_pages
        S, D = max_rows, a.hidden_size
        i32 = dict(dtype=torch.int32, device=d)
        self.pos = torch.zeros(S, **i32)
        self.tok = torch.zeros(S, **i32)
        self.table = torch.full((S, self.max_pages), -1, **i32)
        # the page pool is handed out in a shuffled order (a seeded permutation): pages of a row are not contiguous
        perm = np.random.Generator(np.random.PCG64(seed)).permutation(n_pages).astype(np.int32)
        self.free_list = torch.from_numpy(perm).to(d)
        self.free_top = torch.tensor([n_pages], **i32)
        self.desc = torch.zeros((S, 8), **i32)
        self.parity = torch.zeros(1, **i32)
        self.greedy = torch.zeros(S, **i32)
        self.pairs = torch.zeros((S, 2), **i32)
        self.pairs_all = torch.zeros((model.tp_size, S, 2), **i32)
        bf = dict(dtype=BF16, device=d)
        f32 = dict(dtype=torch.float32, device=d)
        m = model
        self.has_bcsa = "bcsa" in a.mixer_types
        self.indexer = self.has_bcsa and a.bcsa_score == "indexer"
        C = a.bcsa_compress
        self.layers = []
        for mix in a.mixer_types:
            if mix == "kda":
                Cc = 2 * m.Hk * 128 + m.HV * 128
                self.layers.append({"conv": torch.zeros((2, S, 3, Cc), **bf), "S": torch.zeros((S, m.HV, 128, 128), **f32)})
            else:
                st = {"K": torch.zeros((n_pages, m.KVH, PAGE, 128), **bf), "V": torch.zeros((n_pages, m.KVH, PAGE, 128), **bf)}
                if mix == "bcsa":
                    st["PK"] = torch.zeros((n_pages, m.KVH, PAGE // C, 128), **bf)
                    st["PV"] = torch.zeros((n_pages, m.KVH, PAGE // C, 128), **bf)
                    if self.indexer:
                        st["BK"] = torch.zeros((n_pages, PAGE // C, a.bcsa_index_dim), **bf)
                        st["IK"] = torch.zeros((S, C, a.bcsa_index_dim), **bf)
                self.layers.append(st)
        self.keep = max(a.engram_orders) - 1 if a.engram_layers else 0
        self.engram_prev = torch.full((S, max(self.keep, 1)), -1, **i32)
        self.engram_rows = torch.zeros((S, max(len(a.engram_orders), 1)), **i32)
        # ---- activations of one step (fixed addresses: the step is captured as a CUDA graph)
        wid = 0
        for w in m.layers:
            wid = max(wid, w["proj"].N)
        self.H = torch.zeros((S, 4, D), **bf)
        self.hn, self.x_in, self.h = (torch.zeros((S, D), **bf) for _ in range(3))
        self.post, self.res, self.dyn = torch.zeros((S, 4), **f32), torch.zeros((S, 16), **f32), torch.zeros((S, 24), **f32)
        self.proj = torch.zeros((S, wid), **bf)
        self.mix = torch.zeros((S, max(m.HV * 128, m.Hq * 128)), **bf)
        self.r, self.h2, self.hn2, self.mlp = (torch.zeros((S, D), **bf) for _ in range(4))
        self.gu = torch.zeros((S, 2 * m.I), **bf)
        self.act = torch.zeros((S, m.I), **bf)
        self.logits = torch.zeros((S, m.vocab_shard), **bf)
        # activations in the W4 GEMM's input layout (2176 bytes per 64 columns), written by the producing kernels;
        # rows the batch does not use stay zero (cleared whenever the membership changes)
        u8 = dict(dtype=torch.uint8, device=d)
        self.xr_h = torch.zeros(D // 64 * 2176, **u8)
        self.xr_mix = torch.zeros(self.mix.shape[1] // 64 * 2176, **u8)
        self.xr_hn2 = torch.zeros(D // 64 * 2176, **u8)
        self.xr_act = torch.zeros(m.I // 64 * 2176, **u8)
        self.fused_xrec = S <= 16
        self.fuse_boundary = True   # one kernel for combine(layer i) + mix(layer i + 1)
        self.tile_attention = True  # chunk path: attention over tiles of 16 query rows (else one query row at a time)
        self.q = torch.zeros((S, m.Hq, 128), **bf)
        if self.indexer:
            self.qi = torch.zeros((S, a.bcsa_index_heads, a.bcsa_index_dim), **bf)
            self.idxq = torch.zeros((S, a.bcsa_index_heads * a.bcsa_index_dim), **bf)
            self.idxk = torch.zeros((S, a.bcsa_index_dim), **bf)
        self.NS = (1 if self.indexer else m.KVH) if self.has_bcsa else 0
        self.sel = torch.full((S, max(self.NS, 1), max(a.bcsa_topk, 1)), -1, **i32)
        self.nsel = torch.zeros((S, max(self.NS, 1)), **i32)
        self.max_blocks = self.max_pages * (PAGE // C) if self.has_bcsa else 1
        self.sel_scratch = torch.zeros((S, max(self.NS, 1), self.max_blocks), **i32)
        self.nsplit_bcsa, self.nsplit_dense = 16, 64
        if os.environ.get("VK_NSPLIT"):   # tuning: "bcsa,dense"
            self.nsplit_bcsa, self.nsplit_dense = (int(v) for v in os.environ["VK_NSPLIT"].split(","))
        self.part = torch.zeros((S, m.Hq, max(self.nsplit_bcsa, self.nsplit_dense), 130), **f32)
        if a.engram_layers:
            cat = a.engram_dim * len(a.engram_orders)
            self.eng_e = torch.zeros((S, cat), **bf)
            self.eng_val = torch.zeros((S, D), **bf)
        self.orders = (ctypes.c_int * 4)(*(list(a.engram_orders) + [0] * 4)[:4])
        self.geom = {}
        for mix in ("bcsa", "attn"):
            g = _Geom()
            g.Hq, g.KVH, g.D = m.Hq, m.KVH, 128
            bc = mix == "bcsa"
            g.W, g.C, g.topk = (a.bcsa_window, C, a.bcsa_topk) if bc else (0, 1, 1)
            g.IH, g.Di = a.bcsa_index_heads, a.bcsa_index_dim
            g.NS = self.NS if bc else 0
            g.far_tokens = 1 if a.bcsa_far == "tokens" else 0
            g.max_pages, g.n_pages = self.max_pages, n_pages
            self.geom[mix] = g
        self.graphs = {}
        self.kernels_per_step = None
        self.use_graph = True
        self.tp_graph = os.environ.get("VK_TP_GRAPH", "1") == "1"   # capture the NCCL all-reduces into the step's graph
        # Tensor-parallel exchange: inside the consuming kernels over peer memory (default), or NCCL all-reduces between
        # the kernels (VK_TP_FUSED=0: the baseline the fused form is measured against).
        self.ar = None
        if m.tp_size > 1 and os.environ.get("VK_TP_FUSED", "1") == "1":
            from .peer import PeerExchange
            self.ar = PeerExchange(m.group, m.tp_rank, m.tp_size, S, D, 2 * len(m.layers), d)
        self.steps = 0

    # ------------------------------------------------------------------ membership
    @property
    def B(self):
        return len(self.keys)

    def host_pos(self):
        return list(self._pos)

    def row(self, key) -> int:
        return self.keys.index(key)

    def _clear_xrec(self):
        for t in (self.xr_h, self.xr_mix, self.xr_hn2, self.xr_act):
            t.zero_()

    def _sync_rows(self):
        self._clear_xrec()
        self.pos[: self.B] = torch.tensor(self._pos, dtype=torch.int32, device=self.pos.device) if self.B else self.pos[:0]

    def apply(self, leave=(), join=()):
        """Remove the rows of the keys in `leave` (swap-remove: the last row moves into the hole, batch.py:416-431) and
        append one row per item of `join`: a bare key (or (key, None)) starts a fresh sequence at position 0; (key,
        state) continues the sequence a session.State holds (a captured or restored row, the reference's
        join=[(key, b1_cache)], batch.py:432-453): its K/V, pooled blocks and indexer keys are scattered into pages taken
        from the pool, its KDA, conv and Engram state copied into the row's slot. Everything here is enqueued on the
        current stream (page give-back and allocation run as kernels): a membership change does not wait for the GPU."""
        for b in sorted((self.keys.index(k) for k in leave), reverse=True):
            last = self.B - 1
            self._release_pages(b)
            if b != last:
                self._move_row(last, b)
            self._clear_row(last)
            self.keys[b], self._pos[b] = self.keys[last], self._pos[last]
            self.keys.pop()
            self._pos.pop()
        for item in join:
            key, state = item, None
            if isinstance(item, tuple) and len(item) == 2 and (item[1] is None or isinstance(item[1], SS.State)):
                key, state = item
            assert self.B < self.S, "batch is full"
            b = self.B
            self._clear_row(b)
            self.keys.append(key)
            self._pos.append(0)
            if state is not None and state.pos > 0:
                self._put_row(b, state)
        self._sync_rows()

    def release_pages(self, items, reverse):
        """items: (row, first page index, last page index): those table entries go back to the pool on the GPU."""
        if not items:
            return
        dev = self.pos.device
        t = torch.tensor(items, dtype=torch.int32).t().contiguous().to(dev, non_blocking=True)   # [3, n]
        _lib.check(_lib.lib().vk_pages_release(_p(t[0]), _p(t[1]), _p(t[2]), len(items), 1 if reverse else 0, _p(self.table),
                                               self.max_pages, _p(self.free_list), _p(self.free_top), self.n_pages,
                                               torch.cuda.current_stream().cuda_stream), "vk_pages_release")

    def _release_pages(self, b):
        # a row that leaves hands its pages back last first: the next row to grow takes them in the same order
        n = (self._pos[b] + PAGE - 1) // PAGE
        if n:
            self.release_pages([(b, 0, n)], reverse=True)

    def _par(self):
        return self.steps & 1

    def _move_row(self, src, dst):
        par = self._par()
        for st in self.layers:
            if "S" in st:
                st["S"][dst] = st["S"][src]
                st["conv"][par, dst] = st["conv"][par, src]
            elif "IK" in st:
                st["IK"][dst] = st["IK"][src]
        self.table[dst] = self.table[src]
        self.engram_prev[dst] = self.engram_prev[src]

    def _clear_row(self, b):
        for st in self.layers:
            if "S" in st:
                st["S"][b].zero_()
                st["conv"][:, b].zero_()
            elif "IK" in st:
                st["IK"][b].zero_()
        self.table[b] = -1
        self.engram_prev[b] = -1

    def _put_row(self, b, state: SS.State):
        """Row b (cleared, no pages) takes over the sequence of `state`."""
        L = _lib.lib()
        a, dev = self.args, self.pos.device
        P = int(state.pos)
        npg = (P + PAGE - 1) // PAGE
        assert npg <= self.max_pages, "the sequence does not fit a row's page table"
        assert len(state.layers) == len(self.layers) + 1, "the state was captured from another model"
        # pages for positions 0 .. P - 1 of this row only (zero tokens for every other row)
        lens = torch.zeros(self.S, dtype=torch.int32)
        lens[b] = P
        lens = lens.to(dev, non_blocking=True)
        zero = torch.zeros(self.S, dtype=torch.int32, device=dev)
        _lib.check(L.vk_pages_open(_p(zero), _p(lens), _p(self.table), self.max_pages, _p(self.free_list), _p(self.free_top),
                                   self.S, torch.cuda.current_stream().cuda_stream), "vk_pages_open")
        pages = self.table[b, :npg].long()          # (a device tensor: indexing with it needs no host round trip)
        par = self._par()
        C = a.bcsa_compress
        KVH = self.model.KVH

        def to_pages(x, per_page):
            """[1, heads.., n, D] rows by position -> [npg, heads.., per_page, D] (zero padded)."""
            x = x[0]
            n = x.shape[-2]
            pad = npg * per_page - n
            if pad:
                x = torch.cat([x, x.new_zeros(x.shape[:-2] + (pad, x.shape[-1]))], dim=-2)
            x = x.reshape(x.shape[:-2] + (npg, per_page, x.shape[-1]))
            return x.movedim(-3, 0)

        for mix, st, t in zip(a.mixer_types, self.layers, state.layers):
            if mix == "kda":
                assert t[0] == "arrays"
                st["conv"][par, b] = t[1][0].to(dev)
                st["S"][b] = t[2][0].to(dev)
            elif mix == "attn":
                assert t[0] == "kv" and t[1] == P and t[2].shape[1] == KVH
                st["K"][pages] = to_pages(t[2].to(dev)[:, :, :P], PAGE)
                st["V"][pages] = to_pages(t[3].to(dev)[:, :, :P], PAGE)
            else:
                kind, W, Cs, _, offset, nb, k, v, pk, pv, bk, ik = t
                assert kind == "bcsa" and offset == P and W == a.bcsa_window and Cs == C and nb == P // C
                st["K"][pages] = to_pages(k.to(dev)[:, :, :P], PAGE)
                st["V"][pages] = to_pages(v.to(dev)[:, :, :P], PAGE)
                if nb:
                    # (pooled rows of the pages that hold closed blocks; later pages keep what they have: nothing reads
                    # a pooled slot before the block it belongs to has closed)
                    nbp = (nb + PAGE // C - 1) // (PAGE // C)
                    pkp = pk.to(dev)[0][:, :nb]
                    pvp = pv.to(dev)[0][:, :nb]
                    pad = nbp * (PAGE // C) - nb
                    if pad:
                        z = pkp.new_zeros((KVH, pad, pkp.shape[-1]))
                        pkp, pvp = torch.cat([pkp, z], 1), torch.cat([pvp, z], 1)
                    st["PK"][pages[:nbp]] = pkp.reshape(KVH, nbp, PAGE // C, -1).movedim(1, 0)
                    st["PV"][pages[:nbp]] = pvp.reshape(KVH, nbp, PAGE // C, -1).movedim(1, 0)
                    if "BK" in st:
                        bkp = bk.to(dev)[0][:nb]
                        if pad:
                            bkp = torch.cat([bkp, bkp.new_zeros((pad, bkp.shape[-1]))], 0)
                        st["BK"][pages[:nbp]] = bkp.reshape(nbp, PAGE // C, -1)
                if "IK" in st:
                    st["IK"][b] = ik.to(dev)[0]
        eng = state.layers[-1]
        assert eng[0] == "engram"
        if self.keep:
            assert eng[1] == self.keep
            self.engram_prev[b, : self.keep] = eng[2].to(dev)[0]
        self._pos[b] = P

    def attend_splits(self, B, bcsa):
        """KV splits of the decode attention for B rows: about four CTAs per SM in all for the sparse layers (a CTA's fixed
        part, staging Q and resolving its first unit, is a quarter of its life at 16 splits and 16 rows; measured: 4 splits
        10.76 ms per step, 8: 10.80, 16: 10.82), never more than nsplit_bcsa; the dense layer keeps its own count."""
        if not bcsa:
            return self.nsplit_dense
        return max(1, min(self.nsplit_bcsa, -(-592 // (B * self.model.KVH))))

    def capture_row(self, key, dcache=None, logits=None) -> SS.State:
        """Row `key` as a session.State of own copies (batch.py:488-510; layout in volundr_mlx_b200/session.py): the
        position, per layer the KDA conv window and state / the row's K, V (by position), pooled blocks, pooled and
        open-block indexer keys gathered from its pages / the dense layer's K, V, and the Engram id window. `dcache`
        (a drafter's context) and `logits` (of the last position) are carried along as given. Enqueued on the current
        stream; nothing here waits for the GPU."""
        b = self.keys.index(key)
        P = self._pos[b]
        npg = (P + PAGE - 1) // PAGE
        pages = self.table[b, :npg].long()
        a = self.args
        KVH = self.model.KVH
        out = []

        def by_pos(pool, n):
            """[n_pages, KVH, per_page, D] pool -> [1, KVH, n, D] of this row."""
            x = pool[pages]                                   # [npg, KVH, per_page, D]
            return x.movedim(0, 1).reshape(1, KVH, npg * pool.shape[2], x.shape[-1])[:, :, :n].contiguous()

        for mix, st in zip(a.mixer_types, self.layers):
            if mix == "kda":
                out.append(("arrays", st["conv"][self._par(), b: b + 1].clone(), st["S"][b: b + 1].clone()))
            elif mix == "attn":
                out.append(("kv", P, by_pos(st["K"], P), by_pos(st["V"], P)))
            else:
                C = a.bcsa_compress
                nb = P // C
                bk = st["BK"][pages].reshape(1, npg * (PAGE // C), a.bcsa_index_dim)[:, :nb].contiguous() if "BK" in st else None
                ik = st["IK"][b: b + 1].clone() if "IK" in st else None
                out.append(("bcsa", a.bcsa_window, C, 0, P, nb, by_pos(st["K"], P), by_pos(st["V"], P), by_pos(st["PK"], nb),
                            by_pos(st["PV"], nb), bk, ik))
        out.append(("engram", self.keep, self.engram_prev[b: b + 1, : self.keep].clone()))
        state = SS.State(P, out, dcache, None if logits is None else logits.clone())
        state.count_bytes()
        return state

    def row_cache(self, key) -> SS.State:
        """Row `key` as an independent copy that can continue on its own (batch.py:512-515): with a paged cache the
        B = 1 "cache" of a row is its State; join it into any BatchCache of the same model."""
        return self.capture_row(key)

    @property
    def slots_cap(self):
        return self.S

    @property
    def state(self):
        """Every device buffer that holds row state (batch.py:349-356)."""
        out = [self.pos, self.table, self.free_list, self.free_top, self.engram_prev]
        for st in self.layers:
            out += list(st.values())
        return out

    @property
    def nbytes(self):
        return sum(t.numel() * t.element_size() for t in self.state)

    # ------------------------------------------------------------------ synthetic contexts (benchmarks, kernel tests)
    def fill_synthetic(self, keys, ctx_lens, seed=0):
        """Rows that already hold `ctx_lens[i]` tokens: pages allocated from the shuffled pool, K/V ~ N(0,1) (bf16),
        pooled block means computed from them, KDA state ~ N(0, 0.1) fp32, conv state ~ N(0, 1)."""
        assert self.B == 0 and len(keys) <= self.S
        dev = self.pos.device
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed)
        self.keys, self._pos = list(keys), [int(c) for c in ctx_lens]
        top = self.n_pages
        fl = self.free_list.cpu().numpy()
        tab = np.full((self.S, self.max_pages), -1, np.int32)
        for b, P in enumerate(self._pos):
            n = (P + PAGE - 1) // PAGE
            assert n <= self.max_pages and n <= top
            for i in range(n):
                top -= 1
                tab[b, i] = fl[top]
        self.table.copy_(torch.from_numpy(tab))
        self.free_top.fill_(top)
        C = self.args.bcsa_compress
        for st in self.layers:
            if "S" in st:
                st["S"].normal_(0, 0.1, generator=gen)
                st["conv"].normal_(0, 1, generator=gen)
            else:
                for nm in ("K", "V"):
                    buf = st[nm]
                    for i in range(0, self.n_pages, 256):  # chunked: the pool can be many GB
                        buf[i:i + 256].normal_(0, 1, generator=gen)
                if "PK" in st:
                    for i in range(0, self.n_pages, 256):
                        for nm, pn in (("K", "PK"), ("V", "PV")):
                            x = st[nm][i:i + 256].float().reshape(-1, st[nm].shape[1], PAGE // C, C, 128)
                            st[pn][i:i + 256] = (x.sum(3) * (1.0 / C)).to(BF16)
                    if "BK" in st:
                        st["BK"].normal_(0, 1, generator=gen)
                        st["IK"].normal_(0, 1, generator=gen)
        self._sync_rows()
        torch.cuda.synchronize(dev)

    def state_bytes_per_step(self):
        """Bytes of per-row state one decode step must move: KDA state read + written, conv state, K/V rows read."""
        a, m = self.args, self.model
        n = 0
        for mix, st in zip(a.mixer_types, self.layers):
            if mix == "kda":
                n += self.B * (2 * st["S"][0].numel() * 4 + 2 * st["conv"][0, 0].numel() * 2)
            else:
                for P in self._pos:
                    if mix == "attn":
                        keys = P + 1
                    else:
                        W, C = a.bcsa_window, a.bcsa_compress
                        nv = max(0, (P - W + 1) // C)
                        nf = min(nv, a.bcsa_topk)
                        keys = min(P + 1, W) + (nf * C if a.bcsa_far == "tokens" else nf)
                        if nv > a.bcsa_topk:  # scoring reads one pooled key per valid block (per kv head)
                            n += nv * (m.KVH * 128 * 2 if a.bcsa_score == "pooled_key" else a.bcsa_index_dim * 2)
                    n += keys * m.KVH * 128 * 2 * 2
        return n


def _launch_step(model: Model, bc: BatchCache, capture=()):
    """Enqueue one decode step for rows 0..B-1 on the current stream (VolundrModel._fused_layers, volundr.py:939-949;
    DecoderLayer.__call__ :887-906 with split=True; batch.forward, batch.py:518-554)."""
    L = _lib.lib()
    a, B, D = model.args, bc.B, model.args.hidden_size
    st = torch.cuda.current_stream().cuda_stream
    eps = a.rms_norm_eps
    ck = _lib.check
    tp = model.tp_size > 1
    ws = ops.workspace(1 << 26, model.device)
    caps = []

    fx = bc.fused_xrec
    fuse_boundary = bc.fuse_boundary and D % 64 == 0 and D // 8 <= 640 and not capture

    def gemm(x, wt, y, xr=None):
        if fx and xr is not None:
            ck(L.vk_w4_gemm_xrec(_p(wt.packed), _p(xr), _p(y), y.stride(0), B, wt.N, wt.K, _p(ws), ws.numel(), st),
               "vk_w4_gemm_xrec")
        else:
            ck(L.vk_w4_gemm(_p(wt.packed), _p(x), x.stride(0), _p(y), y.stride(0), B, wt.N, wt.K, _p(ws), ws.numel(), st),
               "vk_w4_gemm")

    ar = bc.ar.ref() if bc.ar is not None else None   # exchange inside the consuming kernels

    def allreduce(t):
        if tp and ar is None:
            torch.distributed.all_reduce(t[:B], group=model.group)

    w0 = model.layers[0]
    ck(L.vk_embed(_p(bc.tok), _p(model.embed), _p(w0["mhc_norm"]), _p(bc.H), _p(bc.hn),
                  _p(bc.engram_prev) if a.engram_layers else None, _p(bc.engram_rows), bc.orders,
                  len(a.engram_orders) if a.engram_layers else 0, a.engram_rows, B, D, eps, st), "vk_embed")
    if bc.has_bcsa or "attn" in a.mixer_types:
        ck(L.vk_batch_step_begin(_p(bc.pos), _p(bc.table), bc.max_pages, _p(bc.free_list), _p(bc.free_top), _p(bc.desc), B,
                                 a.bcsa_window if bc.has_bcsa else 0, a.bcsa_compress, a.bcsa_topk, st), "vk_batch_step_begin")
    nl = len(model.layers)
    for i, (w, lst) in enumerate(zip(model.layers, bc.layers)):
        if i in capture:
            caps.append(bc.H[:B, 0].clone())
        if i == 0 or not fuse_boundary:   # (otherwise the previous layer's boundary kernel already did this layer's mix)
            ck(L.vk_mhc_mix_norm(_p(bc.H), _p(bc.hn), _p(w["dyn"]), _p(w["pre_s"]), _p(w["post_s"]), _p(w["res_s"]),
                                 _p(w["ln_in"]), _p(bc.x_in), _p(bc.h), _p(bc.xr_h) if fx else None, _p(bc.post), _p(bc.res),
                                 _p(bc.dyn), B, D, a.mhc_sinkhorn_iters, eps, st), "vk_mhc_mix_norm")
        gemm(bc.h, w["proj"], bc.proj, bc.xr_h)
        if w["mixer"] == "kda":
            nmix = model.HV * 128
            ck(L.vk_kda_step(_p(bc.proj), bc.proj.stride(0), w["off_z"], w["off_fd"], _p(bc.h), _p(w["in_proj_b"]),
                             _p(w["f_up"]), _p(w["conv_w"]), _p(w["A_log"]), _p(w["dt_bias"]), _p(w["gnorm"]),
                             _p(lst["conv"]), _p(bc.parity), lst["conv"][0].numel(), _p(lst["S"]), _p(bc.mix),
                             _p(bc.xr_mix) if fx else None, B, D,
                             model.Hk, model.HV, 128, 128, a.kda_gate_rank, eps, st), "vk_kda_step")
        else:
            bcsa = w["mixer"] == "bcsa"
            g = bc.geom[w["mixer"]]
            nmix = model.Hq * 128
            idx = bcsa and bc.indexer
            if idx:
                ck(L.vk_bf16_gemm(_p(bc.h), D, _p(w["idx_q"]), None, _p(bc.idxq), bc.idxq.stride(0), B,
                                  w["idx_q"].shape[0], D, st), "vk_bf16_gemm")
                ck(L.vk_bf16_gemm(_p(bc.h), D, _p(w["idx_k"]), None, _p(bc.idxk), bc.idxk.stride(0), B,
                                  w["idx_k"].shape[0], D, st), "vk_bf16_gemm")
            ck(L.vk_attn_prep(ctypes.byref(g), _p(bc.proj), bc.proj.stride(0), w["off_k"], w["off_v"],
                              _p(bc.idxq) if idx else None, _p(bc.idxk) if idx else None, _p(w["q_norm"]), _p(w["k_norm"]),
                              _p(w["idx_norm"]) if idx else None, _p(bc.pos), _p(bc.table), _p(bc.q),
                              _p(bc.qi) if idx else None, _p(lst["K"]), _p(lst["V"]), _p(lst.get("PK")), _p(lst.get("PV")),
                              _p(lst.get("BK")), _p(lst.get("IK")), B, model.rope_dims, float(a.rope_theta), eps, st),
               "vk_attn_prep")
            if bcsa:
                ck(L.vk_bcsa_select(ctypes.byref(g), _p(bc.qi) if idx else _p(bc.q), _p(lst["BK"]) if idx else _p(lst["PK"]),
                                    _p(bc.pos), _p(bc.table), _p(bc.sel_scratch), bc.max_blocks, _p(bc.sel), _p(bc.nsel), B,
                                    st), "vk_bcsa_select")
            ck(L.vk_attend_decode(ctypes.byref(g), _p(bc.q), _p(lst["K"]), _p(lst["V"]), _p(lst.get("PK")),
                                  _p(lst.get("PV")), _p(bc.pos), _p(bc.table), _p(bc.sel), _p(bc.nsel), _p(bc.proj),
                                  bc.proj.stride(0), _p(bc.part), bc.attend_splits(B, bcsa), _p(bc.mix),
                                  _p(bc.xr_mix) if fx else None, B, st), "vk_attend_decode")
        mixv = bc.mix[:, :nmix]
        gemm(mixv, w["out"], bc.r, bc.xr_mix)
        allreduce(bc.r)
        ck(L.vk_add_rmsnorm_ar(_p(bc.x_in), _p(bc.r), _p(w["ln_post"]), _p(bc.h2), _p(bc.hn2), _p(bc.xr_hn2) if fx else None,
                               B, D, eps, 1, ar, 2 * i, st),
           "vk_add_rmsnorm_ar")
        gemm(bc.hn2, w["gate_up"], bc.gu, bc.xr_hn2)
        ck(L.vk_silu_mul(_p(bc.gu), None if fx else _p(bc.act), _p(bc.xr_act) if fx else None, B, model.I, bc.gu.stride(0), st),
           "vk_silu_mul")
        gemm(bc.act, w["down"], bc.mlp, bc.xr_act)
        allreduce(bc.mlp)
        eng = "eng_norm" in w
        if eng:
            ptrs, lds, c0 = w["eng_ptrs"]
            ck(L.vk_engram_gather(ptrs.ctypes.data_as(ctypes.c_void_p), lds.ctypes.data_as(ctypes.c_void_p),
                                  c0.ctypes.data_as(ctypes.c_void_p), _p(bc.engram_rows), _p(w["eng_norm"]), _p(bc.eng_e),
                                  B, len(a.engram_orders), a.engram_dim, eps, st), "vk_engram_gather")
            val = bc.eng_e
            if a.engram_value:
                ck(L.vk_bf16_gemm(_p(bc.eng_e), bc.eng_e.stride(0), _p(w["eng_value"]), None, _p(bc.eng_val), D, B, D,
                                  bc.eng_e.shape[1], st), "vk_bf16_gemm")
                val = bc.eng_val
        last = i + 1 == nl
        w_next = model.norm_w if last else model.layers[i + 1]["mhc_norm"]
        if fuse_boundary and not last:
            wn = model.layers[i + 1]
            ck(L.vk_mhc_boundary_ar(_p(bc.H), _p(bc.h2), _p(bc.mlp), _p(bc.x_in), _p(bc.post), _p(bc.res), _p(w_next),
                                    _p(val) if eng else None, _p(w["eng_gate_w"]) if eng else None,
                                    _p(w["eng_gate_b"]) if eng else None, _p(wn["dyn"]), _p(wn["pre_s"]), _p(wn["post_s"]),
                                    _p(wn["res_s"]), _p(wn["ln_in"]), _p(bc.h), _p(bc.xr_h) if fx else None, B, D,
                                    a.mhc_sinkhorn_iters, eps, ar, 2 * i + 1, st), "vk_mhc_boundary_ar")
            continue
        ck(L.vk_mhc_combine_norm_ar(_p(bc.H), _p(bc.h2), _p(bc.mlp), _p(bc.x_in), _p(bc.post), _p(bc.res), _p(w_next),
                                    _p(bc.hn), _p(val) if eng else None, _p(w["eng_gate_w"]) if eng else None,
                                    _p(w["eng_gate_b"]) if eng else None, None, B,
                                    D, 1 if last else 0, eps, ar, 2 * i + 1, st), "vk_mhc_combine_norm_ar")
    V = model.vocab_shard
    if isinstance(model.lm_head, ops.BF16Weight):
        ck(L.vk_bf16_gemm_packed(_p(model.lm_head.packed), _p(bc.hn), D, _p(bc.logits), bc.logits.stride(0), B, V, D, _p(ws),
                                 ws.numel(), st), "vk_bf16_gemm_packed")
    else:
        ck(L.vk_bf16_gemm(_p(bc.hn), D, _p(model.lm_head), None, _p(bc.logits), bc.logits.stride(0), B, V, D, st), "vk_bf16_gemm")
    if not tp:
        ck(L.vk_argmax(_p(bc.logits), bc.logits.stride(0), min(a.vocab_valid, V), _p(bc.greedy), B, st), "vk_argmax")
    else:  # vocabulary-sharded: local (max, index) pairs, all-gather, merge
        n = model.tp_size
        ck(L.vk_argmax_pairs(_p(bc.logits), bc.logits.stride(0), max(0, min(a.vocab_valid - model.vocab0, V)), model.vocab0,
                             _p(bc.pairs), B, st), "vk_argmax_pairs")
        gathered = bc.pairs_all.view(-1)[: n * B * 2].view(n, B, 2)   # contiguous [ranks, B, 2]
        torch.distributed.all_gather_into_tensor(gathered, bc.pairs[:B], group=model.group)
        ck(L.vk_argmax_merge(_p(bc.pairs_all), n, _p(bc.greedy), B, st), "vk_argmax_merge")
    ck(L.vk_batch_step_end(_p(bc.pos), _p(bc.parity), B, st), "vk_batch_step_end")
    if ar is not None:
        ck(L.vk_ar_advance(ar, st), "vk_ar_advance")
    return caps


def forward(model: Model, bc: BatchCache, toks, capture=()):
    """One decode step of every row: toks [B] int32 (tensor on the device, or a host sequence). Returns
    (logits [B, V] bf16, features [B, len(capture) * hidden] or None); the rows' positions advance by one. The
    greedy token of each row (first maximum over the valid vocabulary, scheduler.py:391) is left in bc.greedy[:B].
    The returned tensors are views of step buffers: they are overwritten by the next step."""
    B = bc.B
    assert B > 0
    if not torch.is_tensor(toks):
        toks = torch.tensor(list(toks), dtype=torch.int32)
    bc.tok[:B].copy_(toks.to(torch.int32), non_blocking=True)
    key = (B, tuple(capture))
    if bc.use_graph and not capture and (model.tp_size == 1 or bc.tp_graph):
        g = bc.graphs.get(key)
        if g is None:
            # warm-up launch outside capture is not possible without advancing the rows, so capture directly; the
            # library's kernels need no lazy initialisation beyond the first GEMM's attribute calls
            model_warm(model)
            g = torch.cuda.CUDAGraph()
            n0 = _lib.lib().vk_launch_count(0)
            with torch.cuda.graph(g):
                _launch_step(model, bc, capture)
            bc.kernels_per_step = _lib.lib().vk_launch_count(0) - n0
            bc.graphs[key] = g
            if bc.ar is not None:   # capture takes host time that differs between ranks: line them up before the step
                torch.distributed.barrier(group=model.group)
        g.replay()
        caps = []
    else:
        n0 = _lib.lib().vk_launch_count(0)
        caps = _launch_step(model, bc, capture)
        bc.kernels_per_step = _lib.lib().vk_launch_count(0) - n0
    bc.steps += 1
    bc._pos = [p + 1 for p in bc._pos]
    feats = torch.cat(caps, dim=-1) if caps else None
    return bc.logits[:B], feats


def model_warm(model: Model):
    """Run each GEMM shape once on scratch activations so that one-time function-attribute calls happen outside
    graph capture (once per model object)."""
    if getattr(model, "_vk_warm", False):
        return
    model._vk_warm = True
    d = model.device
    with torch.cuda.device(d):
        _lib.check(_lib.lib().vk_kda_configure(), "vk_kda_configure")
        _lib.check(_lib.lib().vk_attn_configure(), "vk_attn_configure")
    seen = set()
    for w in model.layers:
        for nm in ("proj", "out", "gate_up", "down"):
            wt = w[nm]
            for M in (1, 16):
                if (wt.N, wt.K, M) in seen:
                    continue
                seen.add((wt.N, wt.K, M))
                ops.w4_gemm(torch.zeros((M, wt.K), dtype=BF16, device=d), wt)
    if isinstance(model.lm_head, ops.BF16Weight):
        for M in (1, 16):
            ops.bf16_gemm(torch.zeros((M, model.lm_head.K), dtype=BF16, device=d), model.lm_head)
    if model.tp_size > 1:   # the communicator's first collectives (connection set-up) must not fall inside a capture
        t = torch.zeros((16, model.args.hidden_size), dtype=BF16, device=d)
        torch.distributed.all_reduce(t, group=model.group)
        pr = torch.zeros((16, 2), dtype=torch.int32, device=d)
        al = torch.zeros((model.tp_size, 16, 2), dtype=torch.int32, device=d)
        torch.distributed.all_gather_into_tensor(al, pr, group=model.group)
    torch.cuda.synchronize(d)
