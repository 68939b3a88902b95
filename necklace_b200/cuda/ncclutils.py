"""Pointer / size helpers and the array-level collective wrappers under the reference's
module name (necklace/cuda/ncclutils.py:55-229).  ``nc`` is a group communicator of this
framework (``comm.backend.GroupComm`` / ``comm.symm.TorchGroup`` / ``PeerGroup``) or a
``GroupInfo`` that carries one; ``kn`` (the member count) and ``ndarray`` (the MXNet module the
reference waits on) are accepted and not needed: every call is ordered on the current stream."""
from __future__ import annotations

import numpy as np
import torch

from ..comm import fns as _fns


def tensor_data_ptr(a):
    """Address of the first element: torch tensors, numpy arrays, and objects that expose
    ``data_ptr()`` / ``get_data_p()`` / ``device_ctypes_pointer``."""
    if isinstance(a, torch.Tensor):
        return a.data_ptr()
    if isinstance(a, np.ndarray):
        return a.ctypes.data
    for name in ("data_ptr", "get_data_p"):
        f = getattr(a, name, None)
        if callable(f):
            return int(f())
    p = getattr(a, "device_ctypes_pointer", None)
    if p is not None:
        return int(p.value)
    raise TypeError(f"no buffer address for {type(a).__name__}")


def tensor_size(a):
    """Number of elements."""
    if isinstance(a, torch.Tensor):
        return a.numel()
    return int(getattr(a, "size"))


def tensor_dtype(a):
    """Element type as a torch dtype (numpy arrays are translated)."""
    if isinstance(a, torch.Tensor):
        return a.dtype
    return torch.from_numpy(np.empty(0, dtype=a.dtype)).dtype


def _comm(nc):
    return getattr(nc, "comm", None) or nc


def nccl_all_reduce(og, nc, kn=None, ndarray=None):
    """In-place sum of ``og`` over the group (no division, as in the reference)."""
    if og is None:
        return og
    _comm(nc).all_reduce(og)
    return og


def nccl_all_gather(out, outs, nc, kn=None, ndarray=None):
    """``outs`` = concatenation of every member's ``out``."""
    c = _comm(nc)
    n = out.numel()
    flat = outs.view(-1)
    mine = flat[c.rank * n:(c.rank + 1) * n]
    if mine.data_ptr() != out.data_ptr():
        mine.copy_(out.reshape(-1))
    c.all_gather(flat)
    return outs


def nccl_reduce(buf, root, nc, kn=None, ndarray=None):
    """Sum onto the group's rank ``root`` (the other members' buffers end up summed too)."""
    _comm(nc).all_reduce(buf)
    return buf


def nccl_bcast(buf, root, nc, kn=None, ndarray=None):
    _comm(nc).broadcast(buf, root)
    return buf


def nccl_reduce_scatter(sendbuf, recvbuf, nc, kn=None, ndarray=None):
    """``recvbuf`` = this member's slice of the sum of ``sendbuf`` over the group."""
    _comm(nc).reduce_scatter(sendbuf.view(-1), recvbuf.view(-1))
    return recvbuf


# the two oldest entry points of the reference, same meaning as the wrappers above
seg_cb_nccl_ar = nccl_all_reduce
nccl_out_all_gather = nccl_all_gather

__all__ = ["tensor_data_ptr", "tensor_size", "tensor_dtype", "nccl_all_reduce", "nccl_all_gather",
           "nccl_reduce", "nccl_bcast", "nccl_reduce_scatter", "seg_cb_nccl_ar",
           "nccl_out_all_gather"]
_ = _fns  # the stream-ordered collectives on GroupInfo objects live in comm.fns
