"""The Volundr text model on one B200 (or one tensor-parallel shard of it): parameters in GPU layouts and the
per-layer launch sequence of the batched decode step.

Mirrors the reference's volundr.Model (volundr-mlx/volundr.py:952-994): `Model(args, params)`, `.args`,
`.make_cache()` (here: a BatchCache, batch.py), and the modules' dataflow (DecoderLayer.__call__ :887-906,
VolundrModel._fused_layers :939-949, KDA :388-410, Attention._batched :737-753). Host code only sequences kernels of
libvolundr_b200.so on the current stream; no arithmetic happens in PyTorch.

Linears that share an input are stored as one weight and run as one GEMM: [in_proj_qkv | in_proj_z | f_down],
[q_proj | k_proj | v_proj], [gate_proj | up_proj]. Row-parallel linears (out_proj, o_proj, down_proj) and the
column split of the others follow the tensor-parallel rank (heads and MLP columns), with an all-reduce after
out_proj / o_proj and after down_proj."""
import math

import numpy as np
import torch

from . import _lib, ops
from .synth import ModelArgs

BF16 = torch.bfloat16


def _t(a, device, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(device)
    return t if dtype is None else t.to(dtype)


class _W4:
    """Reference-layout pieces of a 4-bit linear (numpy), sliceable and stackable along the output dimension."""

    def __init__(self, w, s, b):
        self.w, self.s, self.b = w, s, b

    @staticmethod
    def get(p, name):
        return _W4(p[name + ".weight"], p[name + ".scales"], p[name + ".biases"])

    def rows(self, idx):
        return _W4(self.w[idx], self.s[idx], self.b[idx])

    def cols(self, k0, k1, group):
        return _W4(self.w[:, k0 // 8:k1 // 8], self.s[:, k0 // group:k1 // group], self.b[:, k0 // group:k1 // group])

    @staticmethod
    def cat(parts):
        return _W4(np.concatenate([x.w for x in parts]), np.concatenate([x.s for x in parts]),
                   np.concatenate([x.b for x in parts]))

    def to_device(self, device, group):
        w = torch.from_numpy(np.ascontiguousarray(self.w).view(np.int32)).to(device)
        return ops.w4_repack(w, _t(self.s, device, BF16), _t(self.b, device, BF16), group)


class Model:
    def __init__(self, args: ModelArgs, params: dict, device=None, tp_rank: int = 0, tp_size: int = 1, group=None):
        """params: name -> numpy array, reference names (see synth.make_params). `group`: the torch.distributed
        process group of the tensor-parallel ranks (None for one GPU)."""
        self.args = a = args
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.tp_rank, self.tp_size, self.group = tp_rank, tp_size, group
        _lib.lib()  # fail early if the CUDA library is missing
        d = self.device
        g = a.quant_group
        r, n = tp_rank, tp_size
        assert a.head_dim == 128 and a.linear_key_head_dim == 128 and a.linear_value_head_dim == 128, \
            "the CUDA kernels take 128-wide heads"
        assert a.num_key_value_heads % n == 0 and a.linear_num_key_heads % n == 0 and a.intermediate_size % (64 * n) == 0
        Hq, KVH, D = a.num_attention_heads // n, a.num_key_value_heads // n, a.head_dim
        Hk, HV = a.linear_num_key_heads // n, a.linear_num_value_heads // n
        self.Hq, self.KVH, self.Hk, self.HV = Hq, KVH, Hk, HV
        self.I = a.intermediate_size // n
        sl = lambda per, cnt: slice(r * cnt * per, (r + 1) * cnt * per)  # this rank's rows: cnt units of `per`
        self.embed = _t(params["model.embed_tokens.weight"], d, BF16)
        self.norm_w = _t(params["model.norm.weight"], d, BF16)
        V = a.vocab_size
        assert V % n == 0
        self.lm_head = _t(params["lm_head.weight"][r * (V // n):(r + 1) * (V // n)], d, BF16)
        self.layers = []
        self.engram_table = None
        for i, m in enumerate(a.mixer_types):
            L, M = f"model.layers.{i}.", f"model.mhc.{i}."
            w = {"mixer": m}
            w["mhc_norm"] = _t(params[M + "norm.weight"], d, BF16)
            w["dyn"] = _t(params[M + "dyn.weight"], d, BF16)
            w["pre_s"] = _t(params[M + "pre_static"], d, BF16)
            w["post_s"] = _t(params[M + "post_static"], d, BF16)
            w["res_s"] = _t(params[M + "res_static"].reshape(16), d, BF16)
            w["ln_in"] = _t(params[L + "input_layernorm.weight"], d, BF16)
            w["ln_post"] = _t(params[L + "post_attention_layernorm.weight"], d, BF16)
            if m == "kda":
                P = L + "linear_attn."
                KD_full = a.linear_num_key_heads * 128
                qkv = _W4.get(params, P + "in_proj_qkv")
                parts = [qkv.rows(sl(128, Hk)),                                    # q heads of this rank
                         qkv.rows(slice(KD_full + r * Hk * 128, KD_full + (r + 1) * Hk * 128)),
                         qkv.rows(slice(2 * KD_full + r * HV * 128, 2 * KD_full + (r + 1) * HV * 128)),
                         _W4.get(params, P + "in_proj_z").rows(sl(128, HV)),
                         _W4.get(params, P + "f_down")]
                w["proj"] = _W4.cat(parts).to_device(d, g)
                w["off_z"] = 2 * Hk * 128 + HV * 128
                w["off_fd"] = w["off_z"] + HV * 128
                w["in_proj_b"] = _t(params[P + "in_proj_b.weight"][r * HV:(r + 1) * HV], d, BF16)
                w["f_up"] = _t(params[P + "f_up.weight"][sl(128, HV)], d, BF16)
                cw = params[P + "conv1d.weight"]
                cidx = np.r_[np.arange(KD_full)[sl(128, Hk)], KD_full + np.arange(KD_full)[sl(128, Hk)],
                             2 * KD_full + np.arange(a.linear_num_value_heads * 128)[sl(128, HV)]]
                w["conv_w"] = _t(cw[cidx].astype(np.float32), d)
                w["A_log"] = _t(params[P + "A_log"][r * HV:(r + 1) * HV].astype(np.float32), d)
                w["dt_bias"] = _t(params[P + "dt_bias"][sl(128, HV)].astype(np.float32), d)
                w["gnorm"] = _t(params[P + "norm.weight"], d, BF16)
                w["out"] = _W4.get(params, P + "out_proj").cols(r * HV * 128, (r + 1) * HV * 128, g).to_device(d, g)
            else:
                P = L + "self_attn."
                parts = [_W4.get(params, P + "q_proj").rows(sl(2 * D, Hq)),
                         _W4.get(params, P + "k_proj").rows(sl(D, KVH)), _W4.get(params, P + "v_proj").rows(sl(D, KVH))]
                w["proj"] = _W4.cat(parts).to_device(d, g)
                w["off_k"] = Hq * 2 * D
                w["off_v"] = w["off_k"] + KVH * D
                w["q_norm"] = _t(params[P + "q_norm.weight"], d, BF16)
                w["k_norm"] = _t(params[P + "k_norm.weight"], d, BF16)
                if m == "bcsa" and a.bcsa_score == "indexer":
                    w["idx_q"] = _t(params[P + "idx_q.weight"], d, BF16)
                    w["idx_k"] = _t(params[P + "idx_k.weight"], d, BF16)
                    w["idx_norm"] = _t(params[P + "idx_norm.weight"], d, BF16)
                w["out"] = _W4.get(params, P + "o_proj").cols(r * Hq * D, (r + 1) * Hq * D, g).to_device(d, g)
            I = a.intermediate_size
            gate, up = _W4.get(params, L + "mlp.gate_proj"), _W4.get(params, L + "mlp.up_proj")
            w["gate_up"] = _W4.cat([gate.rows(sl(1, self.I)), up.rows(sl(1, self.I))]).to_device(d, g)
            w["down"] = _W4.get(params, L + "mlp.down_proj").cols(r * self.I, (r + 1) * self.I, g).to_device(d, g)
            if i in a.engram_layers:
                E = L + "engram."
                cat = a.engram_dim * len(a.engram_orders)
                if a.engram_shared_table:
                    if self.engram_table is None:
                        self.engram_table = _t(params[E + "table.weight"], d, BF16)
                    w["eng_tables"] = [self.engram_table] * len(a.engram_orders)
                    w["eng_ld"] = [cat] * len(a.engram_orders)
                    w["eng_col0"] = [j * a.engram_dim for j in range(len(a.engram_orders))]
                else:
                    w["eng_tables"] = [_t(params[f"{E}tables.{j}.weight"], d, BF16) for j in range(len(a.engram_orders))]
                    w["eng_ld"] = [a.engram_dim] * len(a.engram_orders)
                    w["eng_col0"] = [0] * len(a.engram_orders)
                w["eng_norm"] = _t(params[E + "norm.weight"], d, BF16)
                w["eng_gate_w"] = _t(params[E + "gate.weight"].reshape(-1), d, BF16)
                w["eng_gate_b"] = _t(params[E + "gate.bias"].reshape(-1), d, BF16)
                if a.engram_value:
                    w["eng_value"] = _t(params[E + "value.weight"], d, BF16)
                w["eng_ptrs"] = (np.array([t.data_ptr() for t in w["eng_tables"]], dtype=np.uint64),
                                 np.array(w["eng_ld"], dtype=np.int32), np.array(w["eng_col0"], dtype=np.int32))
            self.layers.append(w)
        self.rope_dims = int(round(D * a.partial_rotary_factor))
        torch.cuda.synchronize(d)

    def weight_bytes(self):
        """Bytes of parameters one decode step streams (4-bit weights in their packed layout, bf16 linears, lm_head)."""
        n = self.lm_head.numel() * 2
        for w in self.layers:
            for k, v in w.items():
                if isinstance(v, ops.W4Weight):
                    n += v.nbytes
                elif k in ("in_proj_b", "f_up", "dyn", "idx_q", "idx_k", "eng_value"):
                    n += v.numel() * 2
        return n

    def make_cache(self, max_rows: int = 16, n_pages: int = 1024, max_pages_per_row: int = None, seed: int = 0):
        from .batch import BatchCache

        return BatchCache(self, max_rows, n_pages, max_pages_per_row, seed)
