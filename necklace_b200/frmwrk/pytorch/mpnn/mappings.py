"""Autograd mappings of tensor parallelism
(reference: necklace/frmwrk/pytorch/mpnn/mappings.py:25-147):

    copy     forward identity        / backward all-reduce
    reduce   forward all-reduce      / backward identity
    scatter  forward keep my slice of the last dim / backward all-gather
    gather   forward all-gather along the last dim  / backward keep my slice

``gather`` returns a true concatenation along the last dimension (the reference
views rank-major chunks as ``[B, p*d]``, which scrambles rows for B > 1).  Every
collective is ordered on the current stream after the kernel that produced its
operand.
"""
from __future__ import annotations

import torch

from ....comm import fns
from . import initialize as mpu
from .utils import split_tensor_along_last_dim


def _reduce(input_):
    if mpu.get_model_parallel_world_size() == 1:
        return input_
    out = input_.contiguous()
    fns.all_reduce(out, group=mpu.get_model_parallel_group())
    return out


def _split(input_):
    ws = mpu.get_model_parallel_world_size()
    if ws == 1:
        return input_
    return split_tensor_along_last_dim(input_, ws)[mpu.get_model_parallel_rank()].contiguous()


def _gather(input_):
    ws = mpu.get_model_parallel_world_size()
    if ws == 1:
        return input_
    x = input_.contiguous()
    buf = torch.empty((ws,) + tuple(x.shape), dtype=x.dtype, device=x.device)
    fns.all_gather(buf, x, group=mpu.get_model_parallel_group())
    # [p, ..., d] -> [..., p*d]
    return torch.cat(list(buf.unbind(0)), dim=-1)


class _CopyToModelParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input_):
        return input_

    @staticmethod
    def backward(ctx, grad_output):
        return _reduce(grad_output)


class _ReduceFromModelParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input_):
        return _reduce(input_)

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output


class _ScatterToModelParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input_):
        return _split(input_)

    @staticmethod
    def backward(ctx, grad_output):
        return _gather(grad_output)


class _GatherFromModelParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input_):
        return _gather(input_)

    @staticmethod
    def backward(ctx, grad_output):
        return _split(grad_output)


def copy_to_model_parallel_region(input_):
    return _CopyToModelParallelRegion.apply(input_)


def reduce_from_model_parallel_region(input_):
    return _ReduceFromModelParallelRegion.apply(input_)


def scatter_to_model_parallel_region(input_):
    return _ScatterToModelParallelRegion.apply(input_)


def gather_from_model_parallel_region(input_):
    return _GatherFromModelParallelRegion.apply(input_)
