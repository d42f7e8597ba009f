"""Seeded synthetic Volundr-shaped models: argument sets and random-init parameters (NumPy, no checkpoint needed).

The parameter names and shapes are the reference's (volundr.py:293-305, 363-386, 585-592, 635-661, 871-885, 909-916,
952-958); 4-bit linears are stored in the reference's affine layout (codes uint32 [N, K/8], bf16 scales / biases
[N, K/group]). Distributions: codes uniform in [0, 15], scales |N(0, 0.02)| / 8, biases N(0, 0.01) ("free") or
-8 * scale (the reference converter's case, convert.py:11-14, zero-mean weights); everything else as the
reference's tiny test model draws it (tests/tiny.py:27-45)."""
from dataclasses import dataclass, field, asdict
from typing import List

import numpy as np


@dataclass
class ModelArgs:
    """volundr.py:72-113, plus the switches that select the paged benchmark form of BCSA and Engram."""
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
    bcsa_far: str = "pooled"       # "pooled": mean-pooled far K/V (reference) | "tokens": the tokens of chosen pages
    bcsa_score: str = "indexer"    # "indexer": shared indexer heads (reference) | "pooled_key": per kv head
    engram_value: bool = True      # False: the concatenated table rows are hidden_size wide, no value projection
    engram_shared_table: bool = False  # one [rows, dim * orders] table, order i reads columns [i dim, (i+1) dim)
    quant_group: int = 64

    def __post_init__(self):
        if not self.mixer_types:
            raise ValueError("mixer_types is required")
        assert len(self.mixer_types) == self.num_hidden_layers
        assert self.engram_rows & (self.engram_rows - 1) == 0, "Engram hashing keeps only the low bits: rows = 2^k"

    def to_dict(self):
        return asdict(self)


def tiny_args(**kw) -> ModelArgs:
    """The reference's tiny test model (tests/tiny.py:12-20): every mixer kind, Engram, BCSA far regime at short
    lengths (W = 16, C = 4, top-k 3)."""
    d = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=6, num_attention_heads=4, num_key_value_heads=2,
             head_dim=64, vocab_size=300, vocab_valid=290, linear_key_head_dim=32, linear_num_key_heads=2,
             linear_num_value_heads=4, linear_value_head_dim=32, kda_gate_rank=16,
             mixer_types=["kda", "kda", "bcsa", "kda", "bcsa", "attn"], bcsa_window=16, bcsa_compress=4, bcsa_topk=3,
             bcsa_index_heads=2, bcsa_index_dim=32, engram_layers=[1], engram_orders=[2, 3], engram_rows=1024,
             engram_dim=16)
    d.update(kw)
    return ModelArgs(**d)


def small_args(**kw) -> ModelArgs:
    """Smallest shapes the CUDA kernels take (head dims 128, hidden a multiple of 64), reference BCSA semantics."""
    d = dict(hidden_size=256, intermediate_size=512, num_hidden_layers=6, num_attention_heads=4, num_key_value_heads=2,
             head_dim=128, vocab_size=320, vocab_valid=300, linear_key_head_dim=128, linear_num_key_heads=2,
             linear_num_value_heads=4, linear_value_head_dim=128, kda_gate_rank=64,
             mixer_types=["kda", "kda", "bcsa", "kda", "bcsa", "attn"], bcsa_window=16, bcsa_compress=4, bcsa_topk=3,
             bcsa_index_heads=2, bcsa_index_dim=128, engram_layers=[1], engram_orders=[2, 3], engram_rows=1024,
             engram_dim=64)
    d.update(kw)
    return ModelArgs(**d)


def block2_args(**kw) -> ModelArgs:
    """The reduced 2-layer block: 1 KDA + 1 BCSA, hidden 1024, 8 heads x 128 (BCSA 8 q / 2 kv), MLP 4096, BCSA block
    64, top-k 8, paged-token far keys."""
    d = dict(hidden_size=1024, intermediate_size=4096, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2,
             head_dim=128, vocab_size=4096, vocab_valid=4096, linear_key_head_dim=128, linear_num_key_heads=8,
             linear_num_value_heads=8, linear_value_head_dim=128, kda_gate_rank=128, mixer_types=["kda", "bcsa"],
             bcsa_window=128, bcsa_compress=64, bcsa_topk=8, bcsa_far="tokens", bcsa_score="pooled_key",
             engram_layers=[], engram_rows=1024)
    d.update(kw)
    return ModelArgs(**d)


def volundr32b_args(**kw) -> ModelArgs:
    """The 32B-shaped synthetic model: 72 layers (54 KDA, 17 BCSA, 1 dense GQA 40/8), hidden 5120, MLP 22016, vocab
    151936, KDA 40 heads of 128, BCSA 64-token pages with top-32 + a 128-token local window, one 2^20 x 5120 Engram
    table. Layer kinds sit where the reference's synthetic harness puts them (agens-mlx-bench/volundr_synth.py:33-35)."""
    bcsa = {3, 8, 12, 17, 21, 26, 30, 31, 35, 40, 44, 49, 53, 58, 62, 63, 67}
    mixers = ["attn" if i == 71 else "bcsa" if i in bcsa else "kda" for i in range(72)]
    d = dict(hidden_size=5120, intermediate_size=22016, num_hidden_layers=72, num_attention_heads=40,
             num_key_value_heads=8, head_dim=128, vocab_size=151936, vocab_valid=151936, linear_key_head_dim=128,
             linear_num_key_heads=40, linear_num_value_heads=40, linear_value_head_dim=128, kda_gate_rank=128,
             mixer_types=mixers, bcsa_window=128, bcsa_compress=64, bcsa_topk=32, bcsa_far="tokens",
             bcsa_score="pooled_key", engram_layers=[2, 22], engram_orders=[2, 3], engram_rows=1 << 20,
             engram_dim=2560, engram_value=False, engram_shared_table=True)
    d.update(kw)
    return ModelArgs(**d)


def bf(x):
    """float -> the float32 value of its bf16 rounding (nearest even)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    return ((u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))) & np.uint32(0xFFFF0000)).view(np.float32)


def pack_codes(u):
    u = np.asarray(u, dtype=np.uint32)
    w = np.zeros((u.shape[0], u.shape[1] // 8), dtype=np.uint32)
    for j in range(8):
        w |= u[:, j::8] << np.uint32(4 * j)
    return w


# linears the reference keeps in bf16 (convert.py:16-17): lm_head, in_proj_b, mhc.dyn, Engram value / gate, the BCSA
# indexer, plus f_up (bf16 in the release)
_BF16_LINEARS = ("lm_head", "in_proj_b", "dyn", "engram.value", "engram.gate", "idx_q", "idx_k", "f_up")


def linear_shapes(a: ModelArgs):
    """name -> (out, in) of every linear, in the reference's naming."""
    H, I = a.hidden_size, a.intermediate_size
    Hk, HV, K, V = a.linear_num_key_heads, a.linear_num_value_heads, a.linear_key_head_dim, a.linear_value_head_dim
    Hq, KVH, D = a.num_attention_heads, a.num_key_value_heads, a.head_dim
    out = {"lm_head": (a.vocab_size, H)}
    for i, m in enumerate(a.mixer_types):
        L = f"model.layers.{i}."
        out[f"model.mhc.{i}.dyn"] = (2 * a.mhc_streams + a.mhc_streams ** 2, H)
        if m == "kda":
            P = L + "linear_attn."
            out[P + "in_proj_qkv"] = (2 * Hk * K + HV * V, H)
            out[P + "in_proj_z"] = (HV * V, H)
            out[P + "in_proj_b"] = (HV, H)
            out[P + "f_down"] = (a.kda_gate_rank, H)
            out[P + "f_up"] = (HV * K, a.kda_gate_rank)
            out[P + "out_proj"] = (H, HV * V)
        else:
            P = L + "self_attn."
            out[P + "q_proj"] = (Hq * D * 2, H)
            out[P + "k_proj"] = (KVH * D, H)
            out[P + "v_proj"] = (KVH * D, H)
            out[P + "o_proj"] = (H, Hq * D)
            if m == "bcsa" and a.bcsa_score == "indexer":
                out[P + "idx_q"] = (a.bcsa_index_heads * a.bcsa_index_dim, H)
                out[P + "idx_k"] = (a.bcsa_index_dim, H)
        out[L + "mlp.gate_proj"] = (I, H)
        out[L + "mlp.up_proj"] = (I, H)
        out[L + "mlp.down_proj"] = (H, I)
        if i in a.engram_layers:
            out[L + "engram.gate"] = (1, H)
            if a.engram_value:
                out[L + "engram.value"] = (H, a.engram_dim * len(a.engram_orders))
    return out


def make_params(a: ModelArgs, seed: int = 0, quant: bool = True, bias_mode: str = "minus8", weight_std: float = 0.02,
                dtype_round=True, pre_scale: float = 1.0):
    """Random parameters as NumPy arrays (bf16-valued float32 where the reference holds bf16).
    quant=False draws dense N(0, weight_std) matrices for every linear (the fp32 / fp64 validation model)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    r = bf if dtype_round else (lambda x: np.asarray(x, dtype=np.float32))
    p = {}
    H = a.hidden_size
    g = a.quant_group
    for name, (n, k) in linear_shapes(a).items():
        quantize = quant and not any(t in name for t in _BF16_LINEARS) and k % g == 0
        if quantize:
            words = rng.integers(0, 1 << 32, size=(n, k // 8), dtype=np.uint32)  # eight uniform codes per word
            s = bf(np.abs(rng.normal(0, 0.02, size=(n, k // g))) / 8 + 1e-5)
            b = bf(rng.normal(0, 0.01, size=(n, k // g))) if bias_mode == "free" else bf(-8.0 * s)
            p[name + ".weight"], p[name + ".scales"], p[name + ".biases"] = words, s, b
        else:
            p[name + ".weight"] = r(rng.normal(0, weight_std, size=(n, k)))
        if name.endswith("engram.gate"):
            p[name + ".bias"] = r(rng.normal(0, 0.02, size=(1,)))
    p["model.embed_tokens.weight"] = r(rng.normal(0, 1.0, size=(a.vocab_size, H)))
    p["model.norm.weight"] = r(0.1 * rng.normal(size=H))
    Hk, HV, K, V = a.linear_num_key_heads, a.linear_num_value_heads, a.linear_key_head_dim, a.linear_value_head_dim
    C = 2 * Hk * K + HV * V
    n = a.mhc_streams
    for i, m in enumerate(a.mixer_types):
        L = f"model.layers.{i}."
        M = f"model.mhc.{i}."
        p[M + "norm.weight"] = r(1 + 0.1 * rng.normal(size=H))
        p[M + "pre_static"] = r((1.0 + 0.2 * rng.normal(size=n)) * pre_scale)
        p[M + "post_static"] = r(1.0 + 0.2 * rng.normal(size=n))
        p[M + "res_static"] = r(4.0 * np.eye(n) + rng.normal(size=(n, n)))
        p[L + "input_layernorm.weight"] = r(0.1 * rng.normal(size=H))
        p[L + "post_attention_layernorm.weight"] = r(0.1 * rng.normal(size=H))
        if m == "kda":
            P = L + "linear_attn."
            p[P + "conv1d.weight"] = (rng.normal(size=(C, a.linear_conv_kernel_dim)) * 0.5).astype(np.float32)
            p[P + "A_log"] = (rng.normal(size=HV) * 0.3).astype(np.float32)
            p[P + "dt_bias"] = (rng.normal(size=HV * K) * 0.3).astype(np.float32)
            p[P + "norm.weight"] = r(1 + 0.1 * rng.normal(size=V))
        else:
            P = L + "self_attn."
            p[P + "q_norm.weight"] = r(0.1 * rng.normal(size=a.head_dim))
            p[P + "k_norm.weight"] = r(0.1 * rng.normal(size=a.head_dim))
            if m == "bcsa" and a.bcsa_score == "indexer":
                p[P + "idx_norm.weight"] = r(0.1 * rng.normal(size=a.bcsa_index_dim))
        if i in a.engram_layers:
            E = L + "engram."
            cat = a.engram_dim * len(a.engram_orders)
            if a.engram_shared_table:
                key = "model.engram_table.weight"
                if key not in p:
                    p[key] = r(rng.normal(0, 1.0, size=(a.engram_rows, cat)))
                p[E + "table.weight"] = p[key]
            else:
                for j in range(len(a.engram_orders)):
                    p[f"{E}tables.{j}.weight"] = r(rng.normal(0, 1.0, size=(a.engram_rows, a.engram_dim)))
            p[E + "norm.weight"] = r(1 + 0.1 * rng.normal(size=cat))
    return p
