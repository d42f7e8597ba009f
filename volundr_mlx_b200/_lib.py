"""ctypes binding of libvolundr_b200.so (the C ABI declared in include/volundr_b200.h).

There is no CPU or PyTorch fallback behind these calls: a missing library or a non-zero return raises."""
import ctypes
import os
from ctypes import c_int, c_size_t, c_void_p, c_char_p, c_float, c_double
from pathlib import Path

_LIB = None
_PATH = Path(__file__).resolve().parent / "libvolundr_b200.so"

# name -> (restype, argtypes). Every exported symbol of include/volundr_b200.h appears here.
SIGNATURES = {
    "vk_version": (c_int, []),
    "vk_set_pdl": (None, [c_int]),
    "vk_status_fetch": (c_int, [c_void_p, c_void_p]),
    "vk_status_string": (c_char_p, [c_int]),
    "vk_launch_count": (ctypes.c_longlong, [c_int]),
    "vk_w4_packed_bytes": (c_size_t, [c_int, c_int]),
    "vk_w4_repack": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "vk_w4_dequant": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "vk_w4_tile_workspace_bytes": (c_size_t, [c_int, c_int]),
    "vk_w4_tile_workspace_bytes_n": (c_size_t, [c_int, c_int, c_int]),
    "vk_w4_tile_split": (None, [c_int]),
    "vk_w4_gemm_tile": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "vk_w4_tile_force": (c_int, [c_int, c_int]),
    "vk_w4_force_plan": (None, [c_int, c_int]),
    "vk_w4_select": (None, [c_int]),
    "vk_w4_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "vk_w4_gemm": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "vk_bf16_packed_bytes": (c_size_t, [c_int, c_int]),
    "vk_bf16_repack": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "vk_bf16_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "vk_bf16_gemm_packed": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "vk_w4_gemm_xrec": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "vk_embed": (c_int, [c_void_p] * 7 + [c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p]),
    "vk_mhc_mix_norm": (c_int, [c_void_p] * 13 + [c_int, c_int, c_int, c_float, c_void_p]),
    "vk_add_rmsnorm": (c_int, [c_void_p] * 6 + [c_int, c_int, c_float, c_int, c_void_p]),
    "vk_silu_mul": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "vk_engram_gather": (c_int, [c_void_p] * 6 + [c_int, c_int, c_int, c_float, c_void_p]),
    "vk_mhc_combine_norm": (c_int, [c_void_p] * 12 + [c_int, c_int, c_int, c_float, c_void_p]),
    "vk_mhc_boundary_set_cluster": (None, [c_int]),
    "vk_mhc_boundary": (c_int, [c_void_p] * 17 + [c_int, c_int, c_int, c_float, c_void_p]),
    "vk_ar_region_bytes": (c_size_t, [c_int, c_int, c_int]),
    "vk_ar_alloc": (c_int, [c_size_t, c_void_p, c_void_p]),
    "vk_ar_open": (c_int, [c_void_p, c_void_p]),
    "vk_ar_close": (c_int, [c_void_p]),
    "vk_ar_free": (c_int, [c_void_p]),
    "vk_ar_fill": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "vk_ar_advance": (c_int, [c_void_p, c_void_p]),
    "vk_add_rmsnorm_ar": (c_int, [c_void_p] * 6 + [c_int, c_int, c_float, c_int, c_void_p, c_int, c_void_p]),
    "vk_mhc_combine_norm_ar": (c_int, [c_void_p] * 12 + [c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p]),
    "vk_mhc_boundary_ar": (c_int, [c_void_p] * 17 + [c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p]),
    "vk_bf16_gemm": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "vk_argmax": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p]),
    "vk_argmax_pairs": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p]),
    "vk_argmax_merge": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p]),
    "vk_kda_pack_fup": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "vk_kda_configure": (c_int, []),
    "vk_attn_configure": (c_int, []),
    "vk_kda_chunk": (c_int, [c_void_p, c_int, c_int, c_int] + [c_void_p] * 9 + [c_size_t, c_void_p, c_void_p, c_void_p]
                     + [c_int] * 9 + [c_float, c_void_p]),
    "vk_kda_chunk_ragged": (c_int, [c_void_p, c_int, c_int, c_int] + [c_void_p] * 9 + [c_size_t, c_void_p, c_void_p, c_void_p,
                                    c_void_p] + [c_int] * 9 + [c_float, c_void_p]),
    "vk_kda_step": (c_int, [c_void_p, c_int, c_int, c_int] + [c_void_p] * 9 + [c_size_t, c_void_p, c_void_p, c_void_p]
                    + [c_int] * 7 + [c_float, c_void_p]),
    "vk_batch_step_begin": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                    c_void_p]),
    "vk_batch_step_end": (c_int, [c_void_p, c_void_p, c_int, c_void_p]),
    "vk_attn_prep": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int] + [c_void_p] * 15 + [c_int, c_int, c_double, c_float,
                                                                                          c_void_p]),
    "vk_attn_prep_rows": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int] + [c_void_p] * 15 + [c_int, c_int, c_double, c_float,
                                                                                               c_int, c_void_p, c_void_p]),
    "vk_attn_prep_chunk": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int] + [c_void_p] * 15 + [c_int, c_int, c_double, c_float,
                                                                                                c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "vk_pages_open": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "vk_pages_release": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "vk_bcsa_select_scratch_bytes": (c_size_t, [c_void_p, c_int, c_int]),
    "vk_bcsa_select": (c_int, [c_void_p] * 6 + [c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "vk_bcsa_select_static": (c_int, [c_void_p] * 7 + [c_int, c_void_p]),
    "vk_attend_set_tensor_cores": (None, [c_int]),
    "vk_attend_scratch_bytes": (c_size_t, [c_void_p, c_int, c_int]),
    "vk_attend_chunk_smem_bytes": (c_size_t, [c_void_p, c_int]),
    "vk_attend_chunk": (c_int, [c_void_p] * 12 + [c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p]),
    "vk_attend_decode": (c_int, [c_void_p] * 11 + [c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p]),
}


def path() -> Path:
    return _PATH


def lib():
    """The loaded library; raises if it has not been built (python -m volundr_mlx_b200.build)."""
    global _LIB
    if _LIB is None:
        global _PATH
        if os.environ.get("VOLUNDR_B200_LIB"):   # another build of the same library (tuning experiments)
            _PATH = Path(os.environ["VOLUNDR_B200_LIB"])
        if not _PATH.exists():
            raise RuntimeError(f"{_PATH} is missing: build it with `python -m volundr_mlx_b200.build` "
                               "(there is no fallback path)")
        L = ctypes.CDLL(str(_PATH))
        for name, (res, args) in SIGNATURES.items():
            f = getattr(L, name)
            f.restype, f.argtypes = res, args
        _LIB = L
    return _LIB


def check(rc: int, what: str):
    if rc != 0:
        kind = {-1: "invalid argument", -2: "workspace too small",
                -3: "problem larger than the entry point's fixed capacity"}.get(rc, f"CUDA error {rc}")
        raise RuntimeError(f"{what}: {kind}")
