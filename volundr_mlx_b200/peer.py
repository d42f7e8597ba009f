"""Peer-memory region of the in-kernel tensor-parallel exchange (csrc/allreduce.cuh): every rank allocates one region,
the ranks swap CUDA IPC handles through torch.distributed and map each other's regions; the resulting descriptor is
handed to vk_add_rmsnorm_ar / vk_mhc_boundary_ar / vk_mhc_combine_norm_ar. The reference is single-GPU: no counterpart.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib


class ArDesc(ctypes.Structure):
    """vk_ar_desc of include/volundr_b200.h."""
    _fields_ = [("world", ctypes.c_int), ("rank", ctypes.c_int), ("rows", ctypes.c_int), ("row_elems", ctypes.c_int),
                ("calls_per_step", ctypes.c_int), ("spin_limit", ctypes.c_uint), ("slots", ctypes.c_void_p * 8),
                ("step", ctypes.c_void_p)]


def handle_layout(world: int, rank: int, handles: list[bytes]) -> list[bytes | None]:
    """Which handle each rank opens: everybody's but its own (host logic, testable without a GPU)."""
    if len(handles) != world or any(len(h) != 64 for h in handles):
        raise ValueError("one 64-byte handle per rank expected")
    return [None if p == rank else handles[p] for p in range(world)]


class PeerExchange:
    """Owns the local region and the mappings of the peers' regions for one (rows, D, calls_per_step) shape."""

    def __init__(self, group, rank: int, world: int, rows: int, D: int, calls_per_step: int, device):
        import torch.distributed as dist

        L = _lib.lib()
        self.world, self.rank = world, rank
        nbytes = L.vk_ar_region_bytes(world, rows, D)
        if nbytes == 0:
            raise ValueError(f"unsupported exchange shape world={world} rows={rows} D={D}")
        with torch.cuda.device(device):
            base = ctypes.c_void_p()
            handle = ctypes.create_string_buffer(64)
            _lib.check(L.vk_ar_alloc(nbytes, ctypes.byref(base), handle), "vk_ar_alloc")
            self.base = base.value
            handles: list = [None] * world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            self.mapped = []
            bases = (ctypes.c_void_p * 8)()
            for p, h in enumerate(handle_layout(world, rank, handles)):
                if h is None:
                    bases[p] = self.base
                    continue
                ptr = ctypes.c_void_p()
                _lib.check(L.vk_ar_open(ctypes.create_string_buffer(h, 64), ctypes.byref(ptr)), "vk_ar_open")
                self.mapped.append(ptr.value)
                bases[p] = ptr.value
            self.desc = ArDesc()
            _lib.check(L.vk_ar_fill(ctypes.byref(self.desc), world, rank, rows, D, calls_per_step, bases), "vk_ar_fill")
            torch.cuda.synchronize(device)
        dist.barrier(group=group)   # every region is zeroed and mapped before anybody's first push

    def ref(self):
        return ctypes.byref(self.desc)

    def close(self):
        L = _lib.lib()
        for ptr in self.mapped:
            L.vk_ar_close(ptr)
        self.mapped = []
        if self.base:
            L.vk_ar_free(self.base)
            self.base = None
