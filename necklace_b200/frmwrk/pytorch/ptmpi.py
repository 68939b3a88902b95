"""Host-buffer flavour of the parameter / gradient averaging helpers, under the reference's
module name (necklace/frmwrk/pytorch/ptmpi.py:20-260).  The reference copies every tensor to
a numpy buffer and reduces it through an MPI-style communicator object (its ``necklace.pympi``
is absent from its own tree); here the host buffers are reduced through the group's CPU
(gloo) process group when there is one, else staged back to the tensor's device and reduced
there.  ``nc`` is a ``GroupInfo`` (or ``None`` = the data-parallel / main group) as everywhere
in ``ptprms``; results are averages over ``kn`` members."""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from . import ptprms
from .ptprms import (nccl_allreduce_by_buckets, opt_grads_do_nccl_allreduce,  # noqa: F401
                     opt_one_grads_do_nccl_allreduce)
from ...comm import fns as _fns


def _host_allreduce(buf: torch.Tensor, nc) -> torch.Tensor:
    """Sum a CPU tensor over the group in place."""
    group = ptprms._group(nc)
    if group is None or group.world_size == 1 or group.rank < 0:
        return buf
    pg = getattr(getattr(group, "comm", None), "group", None)
    backend = dist.get_backend(pg) if dist.is_initialized() else None
    if backend is not None and "gloo" in str(backend):
        dist.all_reduce(buf, group=pg)
        return buf
    dev = torch.device("cuda", torch.cuda.current_device())
    d = buf.to(dev)
    _fns.all_reduce(d, group=group)
    buf.copy_(d)
    return buf


def nccl_nc_allreduce(nc, p_arr_send, p_arr_recv, sz=None):
    """``p_arr_recv`` = sum over the group of ``p_arr_send`` (tensors; may be the same one)."""
    if p_arr_recv.data_ptr() != p_arr_send.data_ptr():
        p_arr_recv.copy_(p_arr_send)
    _fns.all_reduce(p_arr_recv, group=ptprms._group(nc))
    return p_arr_recv


nccl_pg_allreduce = nccl_nc_allreduce


def nccl_pg_broadcast(pg, p_arr_send, p_arr_recv, sz=None, root=0):
    if p_arr_recv.data_ptr() != p_arr_send.data_ptr():
        p_arr_recv.copy_(p_arr_send)
    _fns.broadcast(p_arr_recv, root, ptprms._group(pg))
    return p_arr_recv


def nccl_pg_reduce(pg, p_arr_send, p_arr_recv, sz=None, root=0):
    if p_arr_recv.data_ptr() != p_arr_send.data_ptr():
        p_arr_recv.copy_(p_arr_send)
    _fns.reduce(p_arr_recv, root, group=ptprms._group(pg))
    return p_arr_recv


def init_params_recvs(model):
    """One host receive buffer per trainable parameter."""
    return {n: torch.zeros(p.shape, dtype=torch.float32) for n, p in model.named_parameters()
            if p.requires_grad and p.dim() >= 1 and p.shape[0] > 0}


def init_opt_grads_recvs(opt):
    """One host receive buffer per parameter of the optimizer (keyed by position)."""
    return {(gi, pi): torch.zeros(p.shape, dtype=torch.float32)
            for gi, g in enumerate(opt.param_groups) for pi, p in enumerate(g["params"])}


def params_do_mpi_allreduce(nc, kn, model, prm_revs=None):
    """Average the weights over the group through host buffers."""
    prm_revs = prm_revs if prm_revs is not None else init_params_recvs(model)
    for name, p in model.named_parameters():
        if not p.requires_grad or name not in prm_revs:
            continue
        buf = prm_revs[name]
        buf.copy_(p.detach().float().cpu())
        _host_allreduce(buf, nc)
        p.data.copy_((buf / float(kn)).to(p.dtype))


def opt_grads_do_mpi_allreduce(nc, kn, opt, prm_revs=None, grad_comp_cfg=None):
    """Average the gradients of the optimizer's parameters through host buffers."""
    prm_revs = prm_revs if prm_revs is not None else init_opt_grads_recvs(opt)
    for gi, g in enumerate(opt.param_groups):
        for pi, p in enumerate(g["params"]):
            if p.grad is None:
                continue
            buf = prm_revs[(gi, pi)]
            buf.copy_(p.grad.detach().float().cpu())
            _host_allreduce(buf, nc)
            p.grad.copy_((buf / float(kn)).to(p.grad.dtype))


_ = np  # host buffers may also be handed in as numpy arrays wrapped by torch.from_numpy
