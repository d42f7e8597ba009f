"""B200-native batched ragged decode step of the Volundr hybrid model (KDA / BCSA / dense GQA on a 4-stream mHC
residual) behind the reference's Python model / batch API. The arithmetic lives in libvolundr_b200.so (hand-written
sm_100a CUDA behind a C ABI); PyTorch supplies device memory, streams and torch.distributed."""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
