"""B200-native Native Sparse Attention operators (sm_100a CUDA behind a C ABI)."""
from . import _lib, ops  # noqa: F401
from ._lib import build  # noqa: F401


def device_status(device=None) -> int:
    """OR of device-side error bits raised by kernels since the last call (0 = none); synchronises."""
    import torch

    stream = torch.cuda.current_stream(device).cuda_stream
    return _lib.lib().nsa_last_device_status(stream)
