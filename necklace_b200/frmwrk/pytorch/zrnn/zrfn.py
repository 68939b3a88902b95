"""Collectives on the ZeRO group and the autograd pair "forward: broadcast the
owner's weights / backward: reduce the gradients to the owner"
(reference: necklace/frmwrk/pytorch/zrnn/zrfn.py:15-129)."""
from __future__ import annotations

import torch

from ....comm import fns, groups as G
from ..mpnn.utils import split_tensor_along_last_dim


def _grp():
    return G.get_nccl_group_zr_or_main()


def zr_pg_all_reduce(input_):
    if G.get_world_size(_grp()) == 1:
        return input_
    fns.all_reduce(input_, group=_grp())
    return input_


def zr_pg_split(input_):
    g = _grp()
    if g.world_size == 1:
        return input_
    return split_tensor_along_last_dim(input_, g.world_size)[g.rank].contiguous()


def zr_pg_all_gather(input_):
    g = _grp()
    if g.world_size == 1:
        return input_
    x = input_.contiguous()
    buf = torch.empty((g.world_size,) + tuple(x.shape), dtype=x.dtype, device=x.device)
    fns.all_gather(buf, x, group=g)
    return torch.cat(list(buf.unbind(0)), dim=-1)


def zr_pg_bcast(input_, root=0):
    fns.broadcast(input_, root, group=_grp())
    return input_


def zr_pg_reduce(input_, root=0):
    fns.reduce(input_, root, group=_grp())
    return input_


class _BcastToZeROParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, weights_, root):
        ctx.root = root
        return zr_pg_bcast(weights_, root)

    @staticmethod
    def backward(ctx, grad_output):
        return zr_pg_reduce(grad_output.contiguous(), ctx.root), None


def bcast_to_zero_parallel_region(weights_, root=0):
    return _BcastToZeROParallelRegion.apply(weights_, root)
