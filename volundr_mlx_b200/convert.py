"""Checkpoint loading: a released Volundr INT4 checkpoint (compressed-tensors `pack-quantized`) or a folder the
reference's converter wrote (MLX safetensors), into the parameter dictionary `volundr.Model(args, params)` takes.

What the reference's convert.py does for the 4-bit linears (convert.py:7-14, :82-137), restated:
  compressed-tensors  weight_packed int32 [n, k/8]: eight nibbles per word, lowest nibble = lowest input index,
                      nibble = q + 8 (q in [-8, 7]); weight_scale bf16 [n, k/g]; w = q * scale
  affine W4           w = scale * u + bias with u = nibble: the packed words are ALREADY the affine codes, and
                      bias = -8 * scale, exact in bf16 (a power-of-two multiple), so bf16(scale * u + bias) equals
                      bf16(q * scale) bit for bit (tests/test_volundr.py:127-156).
  groups              a container that stores scales at a finer group than the linear's type repeats them (g64 scales
                      holding g128 values): they are collapsed when every block repeats one value, kept as stored
                      otherwise (convert.py:104-116).
Everything else is renamed (`model.language_model.` -> `model.`) and passed through: bf16 linears, norms, mHC statics,
Engram tables, embeddings; conv1d weights [C, 1, K] become [C, K] fp32, A_log / dt_bias fp32 (convert.py:221-227).
Only W4 is handled here: the W3 / W2 repacks of the converter have no kernel on this side.

`Model.__init__` then repacks each 4-bit linear into the streaming layout of the GEMM (vk_w4_repack), sliced for its
tensor-parallel rank: loading a checkpoint needs nothing else.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

from .synth import ModelArgs


def _bf16_to_f32(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.float32).numpy()


def collapse_groups(scale: np.ndarray, k: int, group: int):
    """Scales [n, k / g_stored] -> [n, k / group] when every block of `group` inputs repeats one scale; None when the
    stored scales really differ inside a block, or `group` is not a multiple of the stored group."""
    n, cols = scale.shape
    g_stored = k // cols
    if group == g_stored:
        return scale
    if group % g_stored:
        return None
    r = group // g_stored
    s = scale.reshape(n, cols // r, r)
    if not np.all(s == s[..., :1]):
        return None
    return np.ascontiguousarray(s[..., 0])


def convert_linear(packed: np.ndarray, scale: np.ndarray, shape, group: int):
    """compressed-tensors W4 -> (codes uint32 [n, k/8], scales [n, k/group], biases = -8 scales, group): the affine
    layout of convert.py:7-14. `scale` holds bf16 values as float32."""
    n, k = int(shape[0]), int(shape[1])
    assert packed.shape == (n, k // 8), (packed.shape, shape)
    s = collapse_groups(scale, k, group)
    if s is None:
        s, group = scale, k // scale.shape[1]
    if group not in (64, 128):
        raise ValueError(f"group {group}: the GEMM kernels take groups of 64 or 128")
    return packed.view(np.uint32), s.astype(np.float32), (-8.0 * s).astype(np.float32), group


def args_from_config(cfg: dict) -> ModelArgs:
    """ModelArgs from a checkpoint's config.json (the release nests the text model's fields under text_config and
    names the mixers `layer_types`; a converted folder has them at top level as `mixer_types`)."""
    tc = dict(cfg.get("text_config", cfg))
    mixers = tc.get("mixer_types") or tc.get("layer_types")
    rope = tc.get("rope_parameters") or {}
    fields = {f for f in ModelArgs.__dataclass_fields__}
    kw = {k: v for k, v in tc.items() if k in fields}
    kw["mixer_types"] = list(mixers)
    kw.setdefault("num_hidden_layers", len(mixers))
    kw.setdefault("rope_theta", float(rope.get("rope_theta", 1e7)))
    kw.setdefault("partial_rotary_factor", float(rope.get("partial_rotary_factor", 0.25)))
    q = cfg.get("quantization") or cfg.get("quantization_config") or {}
    g0 = q.get("config_groups", {}).get("group_0", {}).get("weights", {})
    kw["quant_group"] = int(q.get("group_size", g0.get("group_size", 128)))
    kw.setdefault("vocab_valid", tc["vocab_size"])
    return ModelArgs(**kw)


def load_params(folder, default_group: int = None):
    """-> (ModelArgs, params): every tensor of the text model under the reference's parameter names, NumPy arrays
    (bf16 tensors as float32 holding the same values). Reads `model.safetensors.index.json` and its shards."""
    from safetensors import safe_open

    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    args = args_from_config(cfg)
    group = default_group or args.quant_group
    wmap = json.loads((folder / "model.safetensors.index.json").read_text())["weight_map"]
    handles = {f: safe_open(str(folder / f), framework="pt") for f in sorted(set(wmap.values()))}
    get = lambda n: handles[wmap[n]].get_tensor(n)
    name_of = lambda n: n.replace("model.language_model.", "model.", 1)
    # the release nests the text model under model.language_model. beside a vision tower; a converted folder has model.
    text = "model.language_model." if any(n.startswith("model.language_model.") for n in wmap) else "model."
    keep = lambda n: n.startswith((text, "lm_head."))
    params = {}
    bases = sorted({n[: -len(".weight_packed")] for n in wmap if n.endswith(".weight_packed") and keep(n)})
    for base in bases:      # the release's container
        packed = get(base + ".weight_packed").numpy()
        scale = _bf16_to_f32(get(base + ".weight_scale"))
        shp = base + ".weight_shape"
        shape = tuple(int(x) for x in get(shp).tolist()) if shp in wmap else (packed.shape[0], packed.shape[1] * 8)
        w, s, b, g = convert_linear(packed, scale, shape, group)
        if g != args.quant_group:
            raise ValueError(f"{base}: group {g}, but the model is built for one group size ({args.quant_group})")
        m = name_of(base)
        params[m + ".weight"], params[m + ".scales"], params[m + ".biases"] = w, s, b
    for n in sorted(wmap):
        if not keep(n) or n.endswith((".weight_packed", ".weight_scale", ".weight_shape")):
            continue
        t = get(n)
        m = name_of(n)
        if n.endswith("conv1d.weight") and t.dim() == 3:
            t = t.reshape(t.shape[0], -1) if t.shape[1] == 1 else t.squeeze(-1)     # [C, 1, K] (torch) or [C, K, 1] (MLX)
        if t.dtype == torch.bfloat16:
            a = _bf16_to_f32(t)
        elif t.dtype in (torch.int32, torch.uint32) or str(t.dtype) == "torch.uint32":
            a = t.numpy().view(np.uint32)
        else:
            a = t.to(torch.float32).numpy() if t.is_floating_point() else t.numpy()
        params[m] = np.ascontiguousarray(a)
    return args, params
