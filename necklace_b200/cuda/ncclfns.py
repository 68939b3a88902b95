"""Collectives on a group with the reference's argument order (necklace/cuda/ncclfns.py:65-260):

    all_gather(output, input_, datatype=None, group=None)
    all_reduce(input_, datatype=None, op=None, group=None)
    broadcast(input_, root=None, datatype=None, group=None)     # root=None: my own group rank
    reduce(input_, root=None, datatype=None, op=None, group=None)

plus the ``pg_*`` forms, which the reference feeds with raw device addresses and an element
count and which take the tensors themselves here (``sz`` is accepted; a send tensor that is
not the receive tensor is copied into it first).  ``datatype`` is accepted and not needed (the
tensor carries its type); ``op`` may be a name (``'sum'``), a value of
``ncclwrp.PYNCCL_REDUCE_OP_MAP`` or ``None`` (= sum).  A rank outside ``group`` returns at
once; everything runs on the caller's current stream.  The implementations live in
``comm.fns``."""
from __future__ import annotations

import torch

from ..comm import fns as _f
from ..comm.fns import barrier, recv, reduce_scatter, send  # noqa: F401
from .ncclwrp import PYNCCL_REDUCE_OP_MAP


def _op(op):
    if op is None:
        return "sum"
    if isinstance(op, str):
        return op
    for name, code in PYNCCL_REDUCE_OP_MAP.items():
        if code == op:
            return name
    raise ValueError(f"unknown reduction operator {op!r}")


def _root(root, group):
    if root is not None:
        return int(root)
    return max(getattr(group, "rank", 0) or 0, 0)


def _pair(send_t, recv_t):
    if not isinstance(send_t, torch.Tensor) or not isinstance(recv_t, torch.Tensor):
        raise TypeError("the pg_* forms take tensors here, not raw device addresses")
    if recv_t.data_ptr() != send_t.data_ptr():
        recv_t.copy_(send_t)
    return recv_t


def all_gather(output, input_, datatype=None, group=None):
    return _f.all_gather(output, input_, group=group)


def pg_all_gather(p_arr_send, p_arr_recv, sz=None, datatype=None, group=None):
    if not isinstance(p_arr_send, torch.Tensor) or not isinstance(p_arr_recv, torch.Tensor):
        raise TypeError("the pg_* forms take tensors here, not raw device addresses")
    return _f.all_gather(p_arr_recv, p_arr_send, group=group)


def all_reduce(input_, datatype=None, op=None, group=None):
    return _f.all_reduce(input_, op=_op(op), group=group)


def pg_all_reduce(p_arr_send, p_arr_recv, sz=None, datatype=None, op=None, group=None):
    return _f.all_reduce(_pair(p_arr_send, p_arr_recv), op=_op(op), group=group)


def broadcast(input_, root=None, datatype=None, group=None):
    return _f.broadcast(input_, _root(root, group), group)


def pg_broadcast(p_arr_send, p_arr_recv, sz=None, root=None, datatype=None, group=None):
    return _f.broadcast(_pair(p_arr_send, p_arr_recv), _root(root, group), group)


def reduce(input_, root=None, datatype=None, op=None, group=None):
    return _f.reduce(input_, _root(root, group), op=_op(op), group=group)


def pg_reduce(p_arr_send, p_arr_recv, sz=None, root=None, datatype=None, op=None, group=None):
    return _f.reduce(_pair(p_arr_send, p_arr_recv), _root(root, group), op=_op(op), group=group)
