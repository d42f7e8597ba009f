"""torch-facing wrappers of the C ABI: tensors in, tensors out, raw pointers and the current stream underneath."""
import torch

from . import _lib

BF16 = torch.bfloat16


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return None if t is None else t.data_ptr()


class W4Weight:
    """An INT4 affine weight in the GEMM's streaming layout (1152-byte chunks of 32 rows x 64 columns)."""

    def __init__(self, packed, N, K, group):
        self.packed, self.N, self.K, self.group = packed, N, K, group

    @property
    def nbytes(self):
        return self.packed.numel()


def w4_repack(w, scales, biases, group=64) -> W4Weight:
    """Reference layout (uint32 [N, K/8] codes as int32 tensor, bf16 scales/biases [N, K/group]) -> W4Weight."""
    L = _lib.lib()
    N, K = w.shape[0], w.shape[1] * 8
    assert w.dtype == torch.int32 and scales.dtype == BF16 and biases.dtype == BF16
    assert scales.shape == (N, K // group) == biases.shape
    packed = torch.empty(L.vk_w4_packed_bytes(N, K), dtype=torch.uint8, device=w.device)
    _lib.check(L.vk_w4_repack(_p(w.contiguous()), _p(scales.contiguous()), _p(biases.contiguous()), N, K, group,
                              _p(packed), _stream()), "vk_w4_repack")
    return W4Weight(packed, N, K, group)


def w4_dequant(w, scales, biases, group=64):
    L = _lib.lib()
    N, K = w.shape[0], w.shape[1] * 8
    out = torch.empty((N, K), dtype=BF16, device=w.device)
    _lib.check(L.vk_w4_dequant(_p(w.contiguous()), _p(scales.contiguous()), _p(biases.contiguous()), N, K, group,
                               _p(out), _stream()), "vk_w4_dequant")
    return out


_ws = {}


def workspace(nbytes, device):
    """One grow-only scratch buffer per device: split-K arrival counters (zero between launches) then the partial
    sums. Allocated outside the step's hot loop."""
    key = str(device)
    buf = _ws.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 1 << 25), dtype=torch.uint8, device=device)
        _ws[key] = buf
    return buf


_tile_ws = {}


def tile_workspace(nbytes, device):
    """Scratch of vk_w4_gemm_tile (arrival counters, zero between launches, activation tiles, partial sums): a buffer of
    its own, since the tile kernel's activation tiles would otherwise land on the streaming kernel's counters."""
    key = str(device)
    buf = _tile_ws.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 1 << 25), dtype=torch.uint8, device=device)
        _tile_ws[key] = buf
    return buf


def w4_gemm(x, wt: W4Weight, out=None):
    """y[M, N] = x[M, K] . dequant(W)^T, bf16 in / out, fp32 accumulation."""
    L = _lib.lib()
    assert x.dtype == BF16 and x.dim() == 2 and x.shape[1] == wt.K and x.stride(1) == 1
    M = x.shape[0]
    if out is None:
        out = torch.empty((M, wt.N), dtype=BF16, device=x.device)
    need = L.vk_w4_workspace_bytes(M, wt.N, wt.K)
    ws = workspace(need, x.device)
    _lib.check(L.vk_w4_gemm(_p(wt.packed), _p(x), x.stride(0), _p(out), out.stride(0), M, wt.N, wt.K, _p(ws),
                            ws.numel(), _stream()), "vk_w4_gemm")
    return out


def w4_gemm_tile(x, wt: W4Weight, out=None):
    """The same product on the tcgen05 tensor cores (tiles of 128 rows): meant for M >= 64."""
    L = _lib.lib()
    assert x.dtype == BF16 and x.dim() == 2 and x.shape[1] == wt.K and x.stride(1) == 1
    M = x.shape[0]
    if out is None:
        out = torch.empty((M, wt.N), dtype=BF16, device=x.device)
    ws = tile_workspace(L.vk_w4_tile_workspace_bytes_n(M, wt.N, wt.K), x.device)
    _lib.check(L.vk_w4_gemm_tile(_p(wt.packed), _p(x), x.stride(0), _p(out), out.stride(0), M, wt.N, wt.K, _p(ws),
                                 ws.numel(), _stream()), "vk_w4_gemm_tile")
    return out


class BF16Weight:
    """A bf16 weight [N, K] in the streaming kernel's fragment order (4096-byte chunks of 32 rows x 64 columns)."""

    def __init__(self, packed, N, K):
        self.packed, self.N, self.K = packed, N, K

    @property
    def nbytes(self):
        return self.packed.numel()


def bf16_repack(W) -> BF16Weight:
    L = _lib.lib()
    N, K = W.shape
    assert W.dtype == BF16 and W.is_contiguous()
    packed = torch.empty(L.vk_bf16_packed_bytes(N, K), dtype=torch.uint8, device=W.device)
    _lib.check(L.vk_bf16_repack(_p(W), N, K, _p(packed), _stream()), "vk_bf16_repack")
    return BF16Weight(packed, N, K)


def bf16_gemm(x, wt: BF16Weight, out=None):
    """y[M, N] = x[M, K] . W^T for a repacked bf16 weight."""
    L = _lib.lib()
    assert x.dtype == BF16 and x.dim() == 2 and x.shape[1] == wt.K and x.stride(1) == 1
    M = x.shape[0]
    if out is None:
        out = torch.empty((M, wt.N), dtype=BF16, device=x.device)
    ws = workspace(L.vk_bf16_workspace_bytes(min(M, 16), wt.N, wt.K), x.device)
    _lib.check(L.vk_bf16_gemm_packed(_p(wt.packed), _p(x), x.stride(0), _p(out), out.stride(0), M, wt.N, wt.K, _p(ws),
                                     ws.numel(), _stream()), "vk_bf16_gemm_packed")
    return out


_status_buf = {}


def check_status(device=None):
    """Read and clear the device status word (synchronises); raises if a kernel recorded an error."""
    L = _lib.lib()
    device = device or torch.device("cuda", torch.cuda.current_device())
    key = str(device)
    if key not in _status_buf:
        _status_buf[key] = torch.zeros(1, dtype=torch.int32, device=device)
    buf = _status_buf[key]
    _lib.check(L.vk_status_fetch(_p(buf), _stream()), "vk_status_fetch")
    code = int(buf.item())
    if code:
        # a wait that ran out may have left a split-K arrival counter behind: put the scratch buffers' heads back to zero
        for pool in (_ws, _tile_ws):
            if key in pool:
                pool[key][: 1 << 14].zero_()
        raise RuntimeError("volundr_b200 device status: " + L.vk_status_string(code).decode())
