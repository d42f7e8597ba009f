"""CPU restatement of one decode step of the Volundr model, row by row, with the reference's rounding points.

Follows the ops branches of volundr-mlx/volundr.py (the path taken when use_kernels() is false, volundr.py:27-29)
and the per-row index arithmetic of volundr-mlx/batch.py. Every row of a batch runs the B = 1 arithmetic
(batch.py:21-24), so a batch step here is a loop over independent `Row` objects.

Two arithmetic modes:
  exact=False  activations are bf16-valued float32 arrays; bf(.) is applied wherever the reference materialises a
               bf16 array (each MLX op on bf16 arrays rounds its result once).
  exact=True   float64, no rounding: used only to validate the dataflow against the reference's own NumPy fp64
               model (volundr-mlx/tests/reference.py), as its test_model_matches_reference_cpu_fp32 does.

BCSA has two parameterisations (ModelArgs.bcsa_far / bcsa_score):
  "pooled"/"indexer"   the reference: far keys are the mean-pooled K/V of closed blocks of C positions, chosen by
                       the indexer scores (volundr.py:705-734, :763-791).
  "tokens"/"pooled_key" the paged 64-token-block form of the benchmark configuration: far keys are the tokens of
                       the chosen blocks; a block's score, per kv head, is the B2 rounding chain with the kv head's
                       query heads as index heads and its mean-pooled key as index key. Not reference behaviour.
"""
from dataclasses import dataclass, field
from typing import List

import numpy as np

from . import w4 as W4
from .numerics import bf

ENGRAM_PRIMES = (1000003, 1000033, 1000037, 1000039, 1000081)  # volundr.py:64


@dataclass
class Args:
    """The fields of the reference's ModelArgs (volundr.py:72-113) plus the benchmark-shape switches."""
    hidden_size: int = 5120
    intermediate_size: int = 17408
    num_hidden_layers: int = 72
    num_attention_heads: int = 24
    num_key_value_heads: int = 4
    head_dim: int = 256
    vocab_size: int = 248320
    vocab_valid: int = 248077
    rms_norm_eps: float = 1e-6
    linear_conv_kernel_dim: int = 4
    linear_key_head_dim: int = 128
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 48
    linear_value_head_dim: int = 128
    kda_gate_rank: int = 128
    mixer_types: List[str] = field(default_factory=list)
    bcsa_window: int = 4096
    bcsa_compress: int = 4
    bcsa_topk: int = 512
    bcsa_index_heads: int = 4
    bcsa_index_dim: int = 128
    engram_layers: List[int] = field(default_factory=list)
    engram_orders: List[int] = field(default_factory=lambda: [2, 3])
    engram_rows: int = 1 << 20
    engram_dim: int = 512
    mhc_streams: int = 4
    mhc_sinkhorn_iters: int = 10
    rope_theta: float = 1e7
    partial_rotary_factor: float = 0.25
    # extensions (not in the reference)
    bcsa_far: str = "pooled"        # "pooled" | "tokens"
    bcsa_score: str = "indexer"     # "indexer" | "pooled_key"
    engram_value: bool = True       # False: concat of table rows == hidden size, no value projection
    quant_group: int = 64


def silu(x):
    with np.errstate(over="ignore"):
        return x / (1 + np.exp(-x))


def sigmoid(x):
    with np.errstate(over="ignore"):
        return 1 / (1 + np.exp(-x))


def tree_dot32(a, b):
    """Dot products over the last axis (length a multiple of 128) in float32 with a fixed order: 32 lanes, lane l
    accumulates elements 4l..4l+3 of each 128-slice in turn with fused multiply-adds, then an xor tree over the
    lanes (offsets 16, 8, 4, 2, 1). Products of bf16 values are exact in float32, so fma and mul+add agree."""
    a = np.asarray(a, dtype=np.float32)
    b = np.asarray(b, dtype=np.float32)
    D = a.shape[-1]
    assert D % 32 == 0 and b.shape[-1] == D
    per = 4 if D % 128 == 0 else D // 32  # (head dims below 128 only occur in the CPU-only tiny model)
    shp = np.broadcast_shapes(a.shape, b.shape)
    p = (a * b).astype(np.float32)
    p = np.broadcast_to(p, shp).reshape(shp[:-1] + (D // (32 * per), 32, per))
    acc = np.zeros(shp[:-1] + (32,), dtype=np.float32)
    for c in range(D // (32 * per)):
        for e in range(per):
            acc = (acc + p[..., c, :, e]).astype(np.float32)
    lanes = np.arange(32)
    for o in (16, 8, 4, 2, 1):
        acc = (acc + acc[..., lanes ^ o]).astype(np.float32)
    return acc[..., 0]


def sinkhorn(logits, iters, dt):
    """sinkhorn_ops (volundr.py:237-243): logits [..., 4, 4] -> doubly stochastic, exp(l - max) then `iters` times
    (rows, columns), each a division by max(sum, 1e-9)."""
    logits = np.asarray(logits, dtype=dt)
    M = np.exp(logits - logits.max(axis=(-1, -2), keepdims=True))
    for _ in range(iters):
        M = M / np.maximum(M.sum(-1, keepdims=True), dt(1e-9))
        M = M / np.maximum(M.sum(-2, keepdims=True), dt(1e-9))
    return M


class Row:
    """Decode state of one sequence: what a B = 1 cache of the reference holds (volundr.py:983-994), kept as full
    histories instead of rings (the window is the last W positions; same values)."""

    def __init__(self, args: Args, dtype):
        a = args
        self.pos = 0
        self.layers = []
        C = 2 * a.linear_num_key_heads * a.linear_key_head_dim + a.linear_num_value_heads * a.linear_value_head_dim
        for m in a.mixer_types:
            if m == "kda":
                self.layers.append({"conv": np.zeros((a.linear_conv_kernel_dim - 1, C), dtype),
                                    "S": np.zeros((a.linear_num_value_heads, a.linear_value_head_dim,
                                                   a.linear_key_head_dim), dtype)})
            elif m == "bcsa":
                self.layers.append({"k": [], "v": [], "pk": [], "pv": [], "bk": [], "ik_open": {}})
            else:
                self.layers.append({"k": [], "v": []})
        self.prev = [-1] * (max(a.engram_orders) - 1 if a.engram_layers else 0)


class Oracle:
    def __init__(self, args: Args, params: dict, exact: bool = False, fast: bool = False, w32: bool = False):
        """fast=True (CPU-baseline timing only): weights dequantised and multiplied in float32 instead of float64.
        w32=True (full-width models): weights dequantised exactly (they are bf16 values, so float32 holds them without
        loss) but kept and multiplied in float32 instead of float64: a quarter of the memory, the product's
        accumulation error (about 1e-6 relative) is far below the bf16 rounding that follows it."""
        self.a, self.p, self.exact, self.fast, self.w32 = args, params, exact, fast, w32
        self.dt = np.float64 if exact else np.float32
        self._wcache = {}

    # ------------------------------------------------------------------ basic ops
    def rnd(self, x):
        return np.asarray(x, dtype=np.float64) if self.exact else bf(x)

    def weight(self, name):
        """Dense [N, K] matrix of linear `name`. A 4-bit linear multiplies by s * u + b as it is, not by its bf16
        rounding: mx.quantized_matmul (volundr.py:185-190) materialises no weights, see oracle.w4.affine; the bf16
        weight bf16(s u + b) is what mx.dequantize returns and is pinned separately (oracle.w4.dequant)."""
        if name not in self._wcache:
            if name + ".scales" in self.p:
                if self.fast:
                    w = W4.dequant_fast(self.p[name + ".weight"], self.p[name + ".scales"], self.p[name + ".biases"],
                                        self.a.quant_group)
                else:
                    w = W4.affine(self.p[name + ".weight"], self.p[name + ".scales"], self.p[name + ".biases"],
                                  self.a.quant_group, np.float32 if self.w32 else np.float64)
            else:
                w = self.p[name + ".weight"]
            self._wcache[name] = np.asarray(w, dtype=np.float32 if (self.fast or self.w32) else np.float64)
        return self._wcache[name]

    def lin(self, x, name):
        """nn.Linear / nn.QuantizedLinear: fp32-accumulated product rounded once (volundr.py:185-190)."""
        W = self.weight(name)
        y = np.asarray(x, dtype=W.dtype) @ W.T
        if name + ".bias" in self.p:
            y = y + np.asarray(self.p[name + ".bias"], dtype=np.float64)
        return self.rnd(y)

    def rms(self, x, w, offset):
        """OffsetRMSNorm / RMSNorm (volundr.py:132-163): x * rsqrt(mean x^2 + eps) * (1 + w | w), one rounding."""
        x = np.asarray(x, dtype=self.dt)
        w = np.asarray(w, dtype=self.dt)
        wf = (1 + w) if offset else w
        inv = 1 / np.sqrt((x * x).mean(-1, keepdims=True) + self.dt(self.a.rms_norm_eps))
        return self.rnd((x * inv) * wf)

    # ------------------------------------------------------------------ Engram
    @staticmethod
    def engram_row(ids, n, rows):
        """Row of the n-gram ending at the last id of `ids` (-1 = none), wrapping uint32 (volundr.py:572-582)."""
        code = 0
        for j in range(n):
            tok = ids[len(ids) - n + j]
            code = (code * ENGRAM_PRIMES[j % len(ENGRAM_PRIMES)] + ((tok + 1) & 0xFFFFFFFF)) & 0xFFFFFFFF
        return code & (rows - 1)

    def engram(self, pre, y, rows):
        """y + sigmoid(gate(y)) * value(norm(concat tables[rows])) (volundr.py:594-597); each bf16 op rounds."""
        a, p = self.a, self.p
        if pre + "table.weight" in p:  # one shared table, order i reads columns [i*dim, (i+1)*dim)
            d = a.engram_dim
            e = np.concatenate([p[pre + "table.weight"][r, i * d:(i + 1) * d] for i, r in enumerate(rows)])
        else:
            e = np.concatenate([p[f"{pre}tables.{i}.weight"][r] for i, r in enumerate(rows)])
        e = self.rms(e, p[pre + "norm.weight"], False)
        g = self.rnd(sigmoid(np.asarray(self.lin(y, pre + "gate"), dtype=self.dt)))
        val = self.lin(e, pre + "value") if a.engram_value else e
        return self.rnd(y + self.rnd(g * val))

    # ------------------------------------------------------------------ mHC
    def mhc_mix(self, i, H, hmean):
        """volundr.py:319-322 with _mhc_params :264-271, sinkhorn_ops :237-243, _mhc_collapse :274-278."""
        p, dt = self.p, self.dt
        m = f"model.mhc.{i}."
        d = np.asarray(self.lin(self.rms(hmean, p[m + "norm.weight"], False), m + "dyn"), dtype=dt)
        pre = self.rnd(np.asarray(p[m + "pre_static"], dt) + d[0:4])
        post = self.rnd(np.asarray(p[m + "post_static"], dt) + d[4:8])
        logits = (np.asarray(p[m + "res_static"], dt).reshape(16) + d[8:24]).reshape(4, 4)
        res = self.rnd(sinkhorn(logits, self.a.mhc_sinkhorn_iters, dt))
        ps = self.rnd(pre[:, None] * H)
        x_in = self.rnd(((ps[0] + ps[1]) + ps[2]) + ps[3])
        return x_in, post, res

    def mhc_combine(self, H, post, res, y, x_in):
        """volundr.py:330-331 (res @ H, bf16 out, fp32 accumulate) and _mhc_combine :281-290."""
        Hd = np.asarray(H, dtype=self.dt)
        mixed = self.rnd(np.asarray(res, self.dt) @ Hd)
        delta = self.rnd(np.asarray(y, self.dt) - x_in)
        upd = self.rnd(np.asarray(post, self.dt)[:, None] * delta[None])
        o = self.rnd(mixed + upd)
        mean = self.rnd((((o[0] + o[1]) + o[2]) + o[3]) * self.dt(0.25))
        return o, mean

    # ------------------------------------------------------------------ KDA
    def kda(self, L, h, st):
        """KDA.__call__ ops branch (volundr.py:418-439) for one token; recurrence as tests/test_volundr.py:103-116."""
        a, dt = self.a, self.dt
        HV, K, V = a.linear_num_value_heads, a.linear_key_head_dim, a.linear_value_head_dim
        qkv = self.lin(h, L + "in_proj_qkv")
        z = np.asarray(self.lin(h, L + "in_proj_z"), dt).reshape(HV, V)
        b = np.asarray(self.lin(h, L + "in_proj_b"), dt)
        aa = np.asarray(self.lin(self.lin(h, L + "f_down"), L + "f_up"), dt).reshape(HV, K)
        out = self.kda_core(L, qkv, z, b, aa, st)
        return self.lin(out.reshape(HV * V), L + "out_proj")

    def kda_core(self, L, qkv, z, b, aa, st):
        """The step from the projections on: conv + SiLU (_conv_silu, volundr.py:351-360), q/k normalisation, decay and
        beta (volundr.py:418-433), the gated delta rule on st["S"] [HV, V, K] (tests/test_volundr.py:103-116) and the
        gated norm (volundr.py:171-174). qkv [C], z [HV, V], b [HV], aa [HV, K] (bf16-valued); returns [HV, V]."""
        a, p, dt = self.a, self.p, self.dt
        Hk, HV, K, V = a.linear_num_key_heads, a.linear_num_value_heads, a.linear_key_head_dim, a.linear_value_head_dim
        conv_in = np.concatenate([st["conv"], np.asarray(qkv, dt)[None]], axis=0)  # [Kc, C]
        st["conv"] = conv_in[1:].copy()
        w = np.asarray(p[L + "conv1d.weight"], dt)  # [C, Kc]
        acc = conv_in[0] * w[:, 0]
        for j in range(1, w.shape[1]):
            acc = acc + conv_in[j] * w[:, j]
        y = np.asarray(self.rnd(silu(acc)), dt)  # _conv_silu, volundr.py:351-360
        q, k, v = y[: Hk * K].reshape(Hk, K), y[Hk * K: 2 * Hk * K].reshape(Hk, K), y[2 * Hk * K:].reshape(HV, V)
        q = q / np.sqrt((q * q).sum(-1, keepdims=True) + dt(1e-6)) * dt(K ** -0.5)
        k = k / np.sqrt((k * k).sum(-1, keepdims=True) + dt(1e-6))
        g = np.exp(-np.exp(np.asarray(p[L + "A_log"], dt))[:, None]
                   * np.logaddexp(aa + np.asarray(p[L + "dt_bias"], dt).reshape(HV, K), 0))
        beta = sigmoid(b)
        S = st["S"]
        o = np.zeros((HV, V), dt)
        for hv in range(HV):
            kh = hv // (HV // Hk)
            S[hv] *= g[hv][None, :]
            S[hv] += np.outer((v[hv] - S[hv] @ k[kh]) * beta[hv], k[kh])
            o[hv] = S[hv] @ q[kh]
        ob = np.asarray(self.rnd(o), dt)
        # _gated_norm (volundr.py:171-174): rms over the value head, * w, * silu(z), one rounding
        wn = np.asarray(p[L + "norm.weight"], dt)
        inv = 1 / np.sqrt((ob * ob).mean(-1, keepdims=True) + dt(a.rms_norm_eps))
        return self.rnd(((ob * inv) * wn) * silu(z))

    # ------------------------------------------------------------------ attention
    def rope(self, x, pos):
        """NeoX rotate-half on the first round(D * factor) dims (volundr.py:651, :663-664; tests/reference.py:71-77)."""
        D = x.shape[-1]
        rd = int(round(D * self.a.partial_rotary_factor))
        inv = self.a.rope_theta ** (-np.arange(0, rd, 2, dtype=np.float64) / rd)
        ang = pos * inv
        cos, sin = np.cos(ang), np.sin(ang)
        x = np.asarray(x, np.float64)
        x1, x2 = x[..., : rd // 2], x[..., rd // 2: rd]
        return self.rnd(np.concatenate([x1 * cos - x2 * sin, x2 * cos + x1 * sin, x[..., rd:]], axis=-1))

    def pool(self, rows):
        """Mean of C bf16 rows in fp32 (added in order), times 1/C, rounded once (BCSACache._pool, volundr.py:470-476)."""
        acc = np.zeros_like(np.asarray(rows[0], self.dt))
        for r in rows:
            acc = (acc + np.asarray(r, self.dt)).astype(self.dt)
        return self.rnd(acc * self.dt(1.0 / len(rows)))

    def block_scores(self, qi, bk):
        """_block_scores (volundr.py:601-606): bf16( bf16( mean_h fp32( bf16(q_h . bk_j) ) ) * scale ).
        qi [IH, Di], bk [nb, Di] -> [nb]. The per-head dot is summed in the fixed order of tree_dot32."""
        IH, Di = qi.shape
        if self.exact:
            e = np.asarray(qi, np.float64) @ np.asarray(bk, np.float64).T  # [IH, nb]
            return e.mean(0) * Di ** -0.5
        e = bf(tree_dot32(qi[:, None, :], bk[None, :, :]))  # [IH, nb]
        s = np.zeros(e.shape[1], np.float32)
        for hh in range(IH):
            s = (s + e[hh]).astype(np.float32)
        s = bf(s * np.float32(1.0 / IH))
        return bf(s * np.float32(Di ** -0.5))

    @staticmethod
    def topk_blocks(s, k):
        """_topk_blocks (volundr.py:609-618): the k largest, ties to the lower index, ascending indices."""
        order = np.argsort(-np.asarray(s, np.float64), kind="stable")[:k]
        return np.sort(order).astype(np.int32)

    def attention(self, L, h, st, pos, bcsa, trace=None):
        """Attention._batched (volundr.py:737-753) for one row at position `pos`; dense = BatchKVCache.attend
        (batch.py:306-316), BCSA = _bcsa_batched (volundr.py:763-791) with BCSAStep's index math (batch.py:100-122)."""
        a, p, dt = self.a, self.p, self.dt
        Hq, KVH, D = a.num_attention_heads, a.num_key_value_heads, a.head_dim
        G = Hq // KVH
        qg = np.asarray(self.lin(h, L + "q_proj"), dt).reshape(Hq, 2 * D)
        q, gate = qg[:, :D], qg[:, D:].reshape(Hq * D)
        q = self.rms(q, p[L + "q_norm.weight"], True)
        k = self.rms(np.asarray(self.lin(h, L + "k_proj"), dt).reshape(KVH, D), p[L + "k_norm.weight"], True)
        v = np.asarray(self.lin(h, L + "v_proj"), dt).reshape(KVH, D)
        q, k = np.asarray(self.rope(q, pos), dt), np.asarray(self.rope(k, pos), dt)
        st["k"].append(k)
        st["v"].append(v)
        scale = D ** -0.5
        if not bcsa:
            lo, far = 0, None
        else:
            W, C, topk = a.bcsa_window, a.bcsa_compress, a.bcsa_topk
            indexer = a.bcsa_score == "indexer"
            if indexer:
                ik = self.rms(self.lin(h, L + "idx_k"), p[L + "idx_norm.weight"], True)
            if (pos + 1) % C == 0:  # the step closes block pos // C (batch.py:243-259)
                blk = range(pos - C + 1, pos + 1)
                st["pk"].append(self.pool([st["k"][t] for t in blk]))
                st["pv"].append(self.pool([st["v"][t] for t in blk]))
                if indexer:
                    st["bk"].append(self.pool([st["ik_open"][t % C] for t in range(pos - C + 1, pos)] + [ik]))
                    st["ik_open"] = {}
            elif indexer:
                st["ik_open"][pos % C] = ik
            nv = max(0, (pos - W + 1) // C)  # blocks lying entirely before the window (batch.py:106)
            lo = max(0, pos - W + 1)
            far = None
            if nv:
                if indexer:
                    qi = np.asarray(self.rms(np.asarray(self.lin(h, L + "idx_q"), dt).reshape(
                        a.bcsa_index_heads, a.bcsa_index_dim), p[L + "idx_norm.weight"], True), dt)
                    if nv > topk:
                        s = self.block_scores(qi, np.stack(st["bk"][:nv]))
                        sel = [self.topk_blocks(s, topk)] * KVH
                    else:
                        sel = [np.arange(nv, dtype=np.int32)] * KVH
                else:  # per kv head: its query heads against its mean-pooled keys
                    sel = []
                    for kv in range(KVH):
                        if nv > topk:
                            s = self.block_scores(q[kv * G:(kv + 1) * G], np.stack([b[kv] for b in st["pk"][:nv]]))
                            sel.append(self.topk_blocks(s, topk))
                        else:
                            sel.append(np.arange(nv, dtype=np.int32))
                far = sel
                if trace is not None:
                    trace.append(("sel", L, pos, [s_.copy() for s_ in sel]))
        out = np.zeros((Hq, D), np.float64)
        for kv in range(KVH):
            K_ = [st["k"][t][kv] for t in range(lo, pos + 1)]
            V_ = [st["v"][t][kv] for t in range(lo, pos + 1)]
            if far is not None:
                if a.bcsa_far == "pooled":
                    K_ += [st["pk"][j][kv] for j in far[kv]]
                    V_ += [st["pv"][j][kv] for j in far[kv]]
                else:
                    C = a.bcsa_compress
                    for j in far[kv]:
                        K_ += [st["k"][t][kv] for t in range(j * C, (j + 1) * C)]
                        V_ += [st["v"][t][kv] for t in range(j * C, (j + 1) * C)]
            K_, V_ = np.asarray(K_, np.float64), np.asarray(V_, np.float64)
            s = (np.asarray(q[kv * G:(kv + 1) * G], np.float64) @ K_.T) * scale
            s = np.exp(s - s.max(-1, keepdims=True))
            out[kv * G:(kv + 1) * G] = (s @ V_) / s.sum(-1, keepdims=True)
        o = np.asarray(self.rnd(out), dt).reshape(Hq * D)
        o = self.rnd(o * sigmoid(np.asarray(gate, dt)))  # _sigmoid_gate, volundr.py:177-179
        return self.lin(o, L + "o_proj")

    # ------------------------------------------------------------------ the step
    def step(self, row: Row, tok: int, trace=None, capture=()):
        """One token of one row: VolundrModel.__call__ (volundr.py:918-937) at L = 1 + lm_head (batch.py:552).
        Returns the logits [vocab]; `capture` layer indices collect the entry stream-0 residual (batch.py:540-541)."""
        a, p, dt = self.a, self.p, self.dt
        x = np.asarray(p["model.embed_tokens.weight"][tok], dt)
        rows = None
        if a.engram_layers:
            full = row.prev + [int(tok)]
            row.prev = full[-(max(a.engram_orders) - 1):]
            rows = [self.engram_row(full, n, a.engram_rows) for n in a.engram_orders]
            if trace is not None:
                trace.append(("engram_rows", rows))
        H = np.stack([x] * a.mhc_streams)
        hmean = x
        caps = []
        for i, mixer in enumerate(a.mixer_types):
            if i in capture:
                caps.append(H[0].copy())
            x_in, post, res = self.mhc_mix(i, H, hmean)
            Lp = f"model.layers.{i}."
            h = self.rms(x_in, p[Lp + "input_layernorm.weight"], True)
            if mixer == "kda":
                r = self.kda(Lp + "linear_attn.", h, row.layers[i])
            else:
                r = self.attention(Lp + "self_attn.", h, row.layers[i], row.pos, mixer == "bcsa", trace)
            h2 = self.rnd(np.asarray(x_in, dt) + r)
            hn = self.rms(h2, p[Lp + "post_attention_layernorm.weight"], True)
            gte = np.asarray(self.lin(hn, Lp + "mlp.gate_proj"), dt)
            up = np.asarray(self.lin(hn, Lp + "mlp.up_proj"), dt)
            m = self.lin(self.rnd(silu(gte) * up), Lp + "mlp.down_proj")  # _silu_mul, volundr.py:166-168
            y = self.rnd(np.asarray(h2, dt) + m)
            if i in a.engram_layers:
                y = self.engram(Lp + "engram.", np.asarray(y, dt), rows)
            H, hmean = self.mhc_combine(H, post, res, y, np.asarray(x_in, dt))
            if trace is not None:
                trace.append(("layer", i, np.asarray(y).copy()))
        row.pos += 1
        logits = self.lin(self.rms(H[0], p["model.norm.weight"], True), "lm_head")
        if capture:
            return logits, np.concatenate(caps)
        return logits

    def new_row(self) -> Row:
        return Row(self.a, self.dt)

    @staticmethod
    def greedy(logits, vocab_valid):
        """First maximum over the valid vocabulary (scheduler.py:391)."""
        return int(np.argmax(np.asarray(logits)[:vocab_valid]))
