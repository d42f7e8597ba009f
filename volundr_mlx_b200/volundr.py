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

from . import _lib, ops, sharding
from .synth import ModelArgs

BF16 = torch.bfloat16


def _t(a, device, dtype=None):
    """numpy array or tensor -> contiguous device tensor (bf16-valued float arrays become bf16 when dtype says so)."""
    t = a if torch.is_tensor(a) else torch.from_numpy(np.ascontiguousarray(a))
    if not torch.is_tensor(a) and t.dtype == torch.uint32:
        t = t.view(torch.int32)
    t = t.to(device)
    return t.contiguous() if dtype is None else t.to(dtype).contiguous()


class _W4:
    """Reference-layout pieces of a 4-bit linear (device tensors), sliceable and stackable along the output rows."""

    def __init__(self, w, s, b):
        self.w, self.s, self.b = w, s, b

    @staticmethod
    def get(p, name, device):
        w = p[name + ".weight"]
        if not torch.is_tensor(w):
            w = torch.from_numpy(np.ascontiguousarray(w).view(np.int32))
        return _W4(w.to(device), _t(p[name + ".scales"], device, BF16), _t(p[name + ".biases"], device, BF16))

    def rows(self, idx):
        return _W4(self.w[idx], self.s[idx], self.b[idx])

    def cols(self, k0, k1, group):
        return _W4(self.w[:, k0 // 8:k1 // 8], self.s[:, k0 // group:k1 // group], self.b[:, k0 // group:k1 // group])

    @staticmethod
    def cat(parts):
        return _W4(torch.cat([x.w for x in parts]), torch.cat([x.s for x in parts]), torch.cat([x.b for x in parts]))

    def to_device(self, device, group):
        return ops.w4_repack(self.w.contiguous(), self.s.contiguous(), self.b.contiguous(), group)


class SynthParams:
    """Random-init parameters generated on the GPU, one tensor per lookup, never all resident at once: the same
    names, shapes and distributions as synth.make_params (codes uniform in [0, 15], scales |N(0, 0.02)| / 8 + 1e-5,
    biases N(0, 0.01) or -8 scale), seeded per name. For models too large to draw on the host."""

    def __init__(self, args: ModelArgs, device, seed: int = 0, bias_mode: str = "free"):
        from . import synth

        self.a, self.device, self.seed, self.bias_mode = args, device, seed, bias_mode
        self.shapes = synth.linear_shapes(args)
        self.bf16_linears = synth._BF16_LINEARS
        self._shared = {}

    def _gen(self, name):
        g = torch.Generator(device=self.device)
        g.manual_seed((hash_name(name) + 1000003 * self.seed) & 0x7FFFFFFFFFFF)
        return g

    def _normal(self, name, shape, std=1.0, mean=0.0, dtype=BF16):
        x = torch.empty(shape, dtype=torch.float32, device=self.device).normal_(mean, std, generator=self._gen(name))
        return x.to(dtype)

    def __contains__(self, name):
        try:
            self[name]
            return True
        except KeyError:
            return False

    def __getitem__(self, name):
        a = self.a
        base, _, leaf = name.rpartition(".")
        if base in self.shapes:
            n, k = self.shapes[base]
            quant = not any(t in base for t in self.bf16_linears) and k % a.quant_group == 0
            if quant:
                if leaf == "weight":
                    lo = torch.randint(0, 1 << 16, (n, k // 8), device=self.device, generator=self._gen(name), dtype=torch.int32)
                    hi = torch.randint(0, 1 << 16, (n, k // 8), device=self.device, generator=self._gen(name + "#hi"), dtype=torch.int32)
                    return lo | (hi << 16)
                s = (self._normal(base + ".scales", (n, k // a.quant_group), 0.02, dtype=torch.float32).abs() / 8 + 1e-5).to(BF16)
                if leaf == "scales":
                    return s
                if leaf == "biases":
                    if self.bias_mode == "free":
                        return self._normal(name, (n, k // a.quant_group), 0.01)
                    return (-8.0 * s.float()).to(BF16)
            elif leaf == "weight":
                return self._normal(name, (n, k), 0.02)
            elif leaf == "bias" and base.endswith("engram.gate"):
                return self._normal(name, (1,), 0.02)
            raise KeyError(name)
        H = a.hidden_size
        Hk, HV = a.linear_num_key_heads, a.linear_num_value_heads
        K, V = a.linear_key_head_dim, a.linear_value_head_dim
        if name == "model.embed_tokens.weight":
            return self._normal(name, (a.vocab_size, H), 1.0)
        if name == "model.norm.weight" or leaf == "weight" and base.endswith(("input_layernorm", "post_attention_layernorm")):
            return self._normal(name, (H,), 0.1)
        if base.endswith(("q_norm", "k_norm")):
            return self._normal(name, (a.head_dim,), 0.1)
        if base.endswith("idx_norm"):
            return self._normal(name, (a.bcsa_index_dim,), 0.1)
        if ".mhc." in name:
            n = a.mhc_streams
            if base.endswith("norm"):
                return self._normal(name, (H,), 0.1, 1.0)
            if leaf in ("pre_static", "post_static"):
                return self._normal(name, (n,), 0.2, 1.0)
            if leaf == "res_static":
                return (4.0 * torch.eye(n, device=self.device) + self._normal(name, (n, n), 1.0, dtype=torch.float32)).to(BF16)
        if "linear_attn" in name:
            C = 2 * Hk * K + HV * V
            if leaf == "weight" and base.endswith("conv1d"):
                return self._normal(name, (C, a.linear_conv_kernel_dim), 0.5, dtype=torch.float32)
            if leaf == "A_log":
                return self._normal(name, (HV,), 0.3, dtype=torch.float32)
            if leaf == "dt_bias":
                return self._normal(name, (HV * K,), 0.3, dtype=torch.float32)
            if base.endswith("linear_attn.norm"):
                return self._normal(name, (V,), 0.1, 1.0)
        if "engram" in name:
            cat = a.engram_dim * len(a.engram_orders)
            if base.endswith("engram.table"):
                if "table" not in self._shared:
                    t = torch.empty((a.engram_rows, cat), dtype=BF16, device=self.device)
                    g = self._gen("model.engram_table.weight")
                    for i in range(0, a.engram_rows, 1 << 16):  # chunked: the fp32 staging copy stays small
                        t[i:i + (1 << 16)] = torch.empty((min(1 << 16, a.engram_rows - i), cat), dtype=torch.float32,
                                                        device=self.device).normal_(0, 1, generator=g).to(BF16)
                    self._shared["table"] = t
                return self._shared["table"]
            if ".tables." in name:
                return self._normal(name, (a.engram_rows, a.engram_dim), 1.0)
            if base.endswith("engram.norm"):
                return self._normal(name, (cat,), 0.1, 1.0)
        raise KeyError(name)


def hash_name(name: str) -> int:
    h = 1469598103934665603
    for ch in name.encode():
        h = ((h ^ ch) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


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
        sharding.check(a, n)
        ix = lambda v: torch.from_numpy(np.asarray(v)).to(d)  # index array -> device
        Hq, KVH, D = a.num_attention_heads // n, a.num_key_value_heads // n, a.head_dim
        Hk, HV = a.linear_num_key_heads // n, a.linear_num_value_heads // n
        self.Hq, self.KVH, self.Hk, self.HV = Hq, KVH, Hk, HV
        self.I = a.intermediate_size // n
        self.embed = _t(params["model.embed_tokens.weight"], d, BF16)
        self.norm_w = _t(params["model.norm.weight"], d, BF16)
        v0, v1 = sharding.vocab_rows(a, r, n)
        self.vocab0 = v0
        head = _t(params["lm_head.weight"], d, BF16)[v0:v1].contiguous()
        self.vocab_shard = head.shape[0]
        self.lm_head = ops.bf16_repack(head) if a.hidden_size % 64 == 0 else head  # streaming layout (tensor cores)
        del head
        self.layers = []
        self.engram_table = None
        for i, m in enumerate(a.mixer_types):
            L, M = f"model.layers.{i}.", f"model.mhc.{i}."
            w = {"mixer": m}
            w["mhc_norm"] = _t(params[M + "norm.weight"], d, BF16)
            w["dyn"] = _t(params[M + "dyn.weight"], d, BF16)
            w["pre_s"] = _t(params[M + "pre_static"], d, BF16)
            w["post_s"] = _t(params[M + "post_static"], d, BF16)
            w["res_s"] = _t(params[M + "res_static"], d, BF16).reshape(16).contiguous()
            w["ln_in"] = _t(params[L + "input_layernorm.weight"], d, BF16)
            w["ln_post"] = _t(params[L + "post_attention_layernorm.weight"], d, BF16)
            if m == "kda":
                P = L + "linear_attn."
                sh = sharding.kda_rows(a, r, n)
                parts = [_W4.get(params, P + "in_proj_qkv", d).rows(ix(sh["qkv"])),   # q | k | v heads of this rank
                         _W4.get(params, P + "in_proj_z", d).rows(ix(sh["z"])),
                         _W4.get(params, P + "f_down", d)]
                w["proj"] = _W4.cat(parts).to_device(d, g)
                w["off_z"] = 2 * Hk * 128 + HV * 128
                w["off_fd"] = w["off_z"] + HV * 128
                w["in_proj_b"] = _t(params[P + "in_proj_b.weight"], d, BF16)[ix(sh["b"])].contiguous()
                fup = _t(params[P + "f_up.weight"], d, BF16)[ix(sh["f_up"])].contiguous()   # [HV*128, rank]
                w["f_up"] = torch.empty_like(fup)                                             # packed for vk_kda_step
                with torch.cuda.device(d):
                    _lib.check(_lib.lib().vk_kda_pack_fup(fup.data_ptr(), w["f_up"].data_ptr(), HV, fup.shape[1],
                                                          torch.cuda.current_stream().cuda_stream), "vk_kda_pack_fup")
                    torch.cuda.current_stream().synchronize()
                w["conv_w"] = _t(params[P + "conv1d.weight"], d, torch.float32)[ix(sh["qkv"])].contiguous()
                w["A_log"] = _t(params[P + "A_log"], d, torch.float32)[ix(sh["b"])].contiguous()
                w["dt_bias"] = _t(params[P + "dt_bias"], d, torch.float32)[ix(sh["f_up"])].contiguous()
                w["gnorm"] = _t(params[P + "norm.weight"], d, BF16)
                w["out"] = _W4.get(params, P + "out_proj", d).cols(*sh["out_cols"], g).to_device(d, g)
            else:
                P = L + "self_attn."
                sh = sharding.attn_rows(a, r, n)
                parts = [_W4.get(params, P + "q_proj", d).rows(ix(sh["q"])),
                         _W4.get(params, P + "k_proj", d).rows(ix(sh["k"])), _W4.get(params, P + "v_proj", d).rows(ix(sh["v"]))]
                w["proj"] = _W4.cat(parts).to_device(d, g)
                w["off_k"] = Hq * 2 * D
                w["off_v"] = w["off_k"] + KVH * D
                w["q_norm"] = _t(params[P + "q_norm.weight"], d, BF16)
                w["k_norm"] = _t(params[P + "k_norm.weight"], d, BF16)
                if m == "bcsa" and a.bcsa_score == "indexer":
                    w["idx_q"] = _t(params[P + "idx_q.weight"], d, BF16)
                    w["idx_k"] = _t(params[P + "idx_k.weight"], d, BF16)
                    w["idx_norm"] = _t(params[P + "idx_norm.weight"], d, BF16)
                w["out"] = _W4.get(params, P + "o_proj", d).cols(*sh["o_cols"], g).to_device(d, g)
            sm = sharding.mlp_rows(a, r, n)
            gate, up = _W4.get(params, L + "mlp.gate_proj", d), _W4.get(params, L + "mlp.up_proj", d)
            w["gate_up"] = _W4.cat([gate.rows(ix(sm["gate"])), up.rows(ix(sm["up"]))]).to_device(d, g)
            w["down"] = _W4.get(params, L + "mlp.down_proj", d).cols(*sm["down_cols"], g).to_device(d, g)
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
                w["eng_gate_w"] = _t(params[E + "gate.weight"], d, BF16).reshape(-1).contiguous()
                w["eng_gate_b"] = _t(params[E + "gate.bias"], d, BF16).reshape(-1).contiguous()
                if a.engram_value:
                    w["eng_value"] = _t(params[E + "value.weight"], d, BF16)
                w["eng_ptrs"] = (np.array([t.data_ptr() for t in w["eng_tables"]], dtype=np.uint64),
                                 np.array(w["eng_ld"], dtype=np.int32), np.array(w["eng_col0"], dtype=np.int32))
            self.layers.append(w)
        self.rope_dims = int(round(D * a.partial_rotary_factor))
        torch.cuda.synchronize(d)

    def weight_bytes(self):
        """Bytes of parameters one decode step streams (4-bit weights in their packed layout, bf16 linears, lm_head)."""
        n = self.vocab_shard * self.args.hidden_size * 2
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
