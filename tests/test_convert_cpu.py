"""Checkpoint loading without a GPU (volundr_mlx_b200.convert): a synthetic release folder in the compressed-tensors
layout the reference's converter reads (convert.py:7-14: int32 words of eight nibbles q + 8, bf16 scales, here stored
at half the linear's group with every scale repeated) comes back as the affine W4 parameters it was made from, bias = -8
scale, and the oracle gives the same logits from the loaded parameters as from the originals; the dequantised weights
equal bf16(q * scale) bit for bit (the reference's own check, convert.py:140-153, tests/test_volundr.py:127-156)."""
import json

import numpy as np
import torch

from oracle import w4 as OW
from oracle.model import Oracle
from oracle.numerics import bf, bf_bits
from volundr_mlx_b200 import convert as CV, synth


def _write_release(folder, args, params):
    from safetensors.torch import save_file

    tensors = {}
    pre = lambda n: n if n.startswith("lm_head.") else n.replace("model.", "model.language_model.", 1)
    bases = {n[: -len(".scales")] for n in params if n.endswith(".scales")}
    for base in sorted(bases):
        w, s = params[base + ".weight"], params[base + ".scales"]
        tensors[pre(base) + ".weight_packed"] = torch.from_numpy(w.view(np.int32).copy())
        tensors[pre(base) + ".weight_scale"] = torch.from_numpy(np.repeat(s, 2, axis=1).copy()).to(torch.bfloat16)   # g / 2, repeated
        tensors[pre(base) + ".weight_shape"] = torch.tensor([w.shape[0], w.shape[1] * 8], dtype=torch.int64)
    for n, a in params.items():
        if any(n.startswith(b + ".") for b in bases) or n == "model.engram_table.weight":
            continue
        t = torch.from_numpy(np.ascontiguousarray(a))
        if n.endswith("conv1d.weight"):
            t = t.reshape(t.shape[0], 1, t.shape[1])                     # torch depthwise layout
        elif not n.endswith((".A_log", ".dt_bias")):
            t = t.to(torch.bfloat16)
        tensors[pre(n)] = t
    tensors["model.visual.patch_embed.weight"] = torch.zeros(4, 4)      # (not part of the text model: must be ignored)
    names = sorted(tensors)
    half = len(names) // 2
    shards = {"model-00001.safetensors": names[:half], "model-00002.safetensors": names[half:]}
    wmap = {}
    for f, ns in shards.items():
        save_file({n: tensors[n].contiguous() for n in ns}, str(folder / f))
        wmap.update({n: f for n in ns})
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wmap}))
    tc = {k: v for k, v in args.to_dict().items() if k not in ("mixer_types", "quant_group", "rope_theta", "partial_rotary_factor")}
    tc["layer_types"] = args.mixer_types
    tc["rope_parameters"] = {"rope_theta": args.rope_theta, "partial_rotary_factor": args.partial_rotary_factor}
    cfg = {"text_config": tc, "quantization_config": {"config_groups": {"group_0": {"weights": {"num_bits": 4, "group_size": args.quant_group}}}}}
    (folder / "config.json").write_text(json.dumps(cfg))


def test_release_folder_round_trip(tmp_path):
    args = synth.tiny_args()
    params = synth.make_params(args, seed=5, quant=True, bias_mode="minus8")
    _write_release(tmp_path, args, params)
    args2, loaded = CV.load_params(tmp_path)
    assert args2.to_dict() == args.to_dict()
    assert set(loaded) == set(params) - {"model.engram_table.weight"}
    for n, a in loaded.items():
        want = params[n]
        assert a.shape == want.shape and np.array_equal(a.view(np.uint8) if a.dtype != want.dtype else a, want.view(np.uint8) if a.dtype != want.dtype else want), n
    assert loaded["model.layers.0.linear_attn.conv1d.weight"].dtype == np.float32
    # dequantised weights == bf16(q * scale), bit for bit
    base = "model.layers.0.mlp.gate_proj"
    w, s, b = loaded[base + ".weight"], loaded[base + ".scales"], loaded[base + ".biases"]
    q = OW.unpack_codes(w, w.shape[1] * 8).astype(np.float32) - 8
    assert np.array_equal(bf_bits(OW.dequant(w, s, b, args.quant_group)), bf_bits(bf(q * np.repeat(s, args.quant_group, axis=1))))
    # the oracle cannot tell the loaded parameters from the originals
    ids = [3, 17, 250, 9, 9, 41]
    a_, b_ = Oracle(args, params), Oracle(args2, loaded)
    ra, rb = a_.new_row(), b_.new_row()
    for t in ids:
        assert np.array_equal(a_.step(ra, t), b_.step(rb, t))


def test_scales_that_differ_inside_a_group_are_kept_as_stored():
    rng = np.random.default_rng(0)
    n, k = 8, 256
    packed = rng.integers(0, 1 << 32, size=(n, k // 8), dtype=np.uint32).view(np.int32)
    s64 = bf(np.abs(rng.normal(0, 0.01, size=(n, k // 64))) + 1e-4)
    w, s, b, g = CV.convert_linear(packed, s64, (n, k), 128)       # asked for g128, stored g64 with distinct values
    assert g == 64 and np.array_equal(s, s64) and np.array_equal(b, -8 * s64)
    w, s, b, g = CV.convert_linear(packed, np.repeat(s64[:, ::2], 2, axis=1), (n, k), 128)
    assert g == 128 and s.shape == (n, 2)
