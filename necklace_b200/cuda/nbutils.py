"""Device helpers under the reference's module name (necklace/cuda/nbutils.py:11-39).  The
reference does these through ``numba.cuda``; here they are the torch equivalents, so the
names user scripts call keep working without numba."""
from __future__ import annotations

import ctypes

import numpy as np
import torch


def cuda_select_device(dev_i):
    """Make GPU ``dev_i`` current (no-op without a GPU)."""
    if torch.cuda.is_available():
        torch.cuda.set_device(int(dev_i))
    return dev_i


def cuda_current_context():
    """The current device as a ``torch.device`` (``cpu`` without a GPU)."""
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def cuda_stream():
    """A new stream on the current device (``None`` without a GPU)."""
    return torch.cuda.Stream() if torch.cuda.is_available() else None


def cuda_to_device(A, stream=None):
    """Copy a host array (numpy or tensor) to the current device, on ``stream`` if given."""
    t = torch.from_numpy(np.ascontiguousarray(A)) if isinstance(A, np.ndarray) else A
    if not torch.cuda.is_available():
        return t.clone()
    if stream is None:
        return t.cuda()
    with torch.cuda.stream(stream):
        return t.pin_memory().cuda(non_blocking=True)


def cuda_devarr_c_void_p(d_arr):
    """The buffer address of a device (or host) tensor as ``ctypes.c_void_p``."""
    return ctypes.c_void_p(int(d_arr.data_ptr()))
