"""Tensor parallelism on the fused GEMM + collective kernels (sequence-parallel layout).

Activations between tensor-parallel regions are kept row-sharded (``[tokens/p, C]`` per
rank).  A column-parallel linear is then "all-gather rows, multiply by my weight
columns" and a row-parallel linear "multiply, reduce-scatter rows":

    ColumnParallel   fwd  Y   = AG(X) W_r^T          one kernel: ``PeerGroup.ag_gemm``
                     bwd  dX  = RS(dY W_r)           one kernel: ``PeerGroup.gemm_rs``
                          dW_r = dY^T AG(X)
    RowParallel      fwd  Y_r = RS(X W_r^T) (+b,+res) one kernel: ``PeerGroup.gemm_rs``
                     bwd  dX  = AG(dY_r) W_r         one kernel: ``PeerGroup.ag_gemm``
                          dW_r = AG(dY_r)^T X

so every collective of the reference's Megatron-style layers
(necklace/frmwrk/pytorch/mpnn/mappings.py:25-82, layers.py:239-249, :314-328) overlaps the
tensor-core work of the GEMM it belongs to, tile by tile, instead of running as a separate
blocking NCCL call.  ``group`` is a ``PeerGroup``; with one rank the plain GEMM is used.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops.gemm import _deliver_grad, colsum, gemm


class _Bufs:
    """Per-group gather buffers in the symmetric heap, keyed by shape (allocated once)."""

    def __init__(self):
        self.d = {}

    def get(self, group, rows, cols, tag):
        key = (id(group), rows, cols, tag)
        t = self.d.get(key)
        if t is None:
            t = group.heap.alloc(rows * cols, torch.bfloat16).view(rows, cols)
            self.d[key] = t
        return t


_BUFS = _Bufs()


class AGLinearFn(torch.autograd.Function):
    """``y[M, N_r] = all_gather_rows(x_shard)[M, K] @ w_r[N_r, K]^T (+ bias)``"""

    @staticmethod
    def forward(ctx, x_shard, w, bias, group):
        p, r = group.world, group.rank
        R, K = x_shard.shape
        ctx.group = group
        if p == 1:
            y = gemm(x_shard, w, bias=bias)
            ctx.save_for_backward(x_shard, w)
            ctx.b_ref = bias
            return y
        xf = _BUFS.get(group, p * R, K, "ag_fwd")
        xf[r * R:(r + 1) * R].copy_(x_shard)
        y = group.ag_gemm(xf, w, bias=bias)
        ctx.save_for_backward(xf.clone(), w)   # gathered input, needed by the weight gradient
        ctx.b_ref = bias
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, w = ctx.saved_tensors
        group = ctx.group
        dy = dy.contiguous()
        if group.world == 1:
            dx = gemm(dy, w, b_mn=True)
        else:
            dx = group.gemm_rs(dy, w, b_mn=True)          # [M/p, K]
        dw = _deliver_grad(w, lambda out, acc: gemm(dy, x_full, a_mn=True, b_mn=True, out=out,
                                                    accumulate=acc))
        db = None
        if ctx.b_ref is not None:
            db = _deliver_grad(ctx.b_ref, lambda out, acc: colsum(dy, out, acc))
        return dx, dw, db, None


class LinearRSFn(torch.autograd.Function):
    """``y_shard[M/p, N] = reduce_scatter_rows(x[M, K_r] @ w_r[N, K_r]^T) (+ bias + residual)``"""

    @staticmethod
    def forward(ctx, x, w, bias, residual, group):
        ctx.group = group
        ctx.save_for_backward(x, w)
        ctx.b_ref, ctx.has_res = bias, residual is not None
        if group.world == 1:
            return gemm(x, w, bias=bias, res=residual)
        return group.gemm_rs(x.contiguous(), w, bias=bias, res=residual)

    @staticmethod
    def backward(ctx, dy_shard):
        x, w = ctx.saved_tensors
        group = ctx.group
        p, r = group.world, group.rank
        dy_shard = dy_shard.contiguous()
        if p == 1:
            dy_full = dy_shard
            dx = gemm(dy_full, w, b_mn=True)
        else:
            R, N = dy_shard.shape
            dyf = _BUFS.get(group, p * R, N, "ag_bwd")
            dyf[r * R:(r + 1) * R].copy_(dy_shard)
            dx = group.ag_gemm(dyf, w, b_mn=True)         # [M, K_r]; also fills dyf
            dy_full = dyf
        dw = _deliver_grad(w, lambda out, acc: gemm(dy_full, x, a_mn=True, b_mn=True, out=out,
                                                    accumulate=acc))
        db = None
        if ctx.b_ref is not None:
            # bias is added once after the reduction: its gradient is the column sum of the
            # local rows, summed over ranks by the data-/tensor-parallel gradient reduction
            db = _deliver_grad(ctx.b_ref, lambda out, acc: colsum(dy_shard, out, acc))
        dres = dy_shard if ctx.has_res else None
        return dx, dw, db, dres, None


def ag_linear(x_shard, w, bias, group):
    return AGLinearFn.apply(x_shard, w, bias, group)


def linear_rs(x, w, bias, residual, group):
    return LinearRSFn.apply(x, w, bias, residual, group)


class SPColumnParallelLinear(nn.Module):
    """Column-parallel linear over row-sharded input (fused all-gather -> GEMM)."""

    def __init__(self, in_features, out_features, group, bias=True, dtype=torch.bfloat16,
                 device=None, seed=1234, std=0.02):
        super().__init__()
        p, r = group.world, group.rank
        assert out_features % p == 0
        g = torch.Generator().manual_seed(seed)
        full = torch.randn(out_features, in_features, generator=g) * std
        self.group = group
        self.weight = nn.Parameter(full.chunk(p, 0)[r].contiguous().to(dtype).to(device))
        self.bias = nn.Parameter(torch.zeros(out_features // p, dtype=dtype, device=device)) \
            if bias else None
        self.weight.model_parallel, self.weight.partition_dim = True, 0
        if self.bias is not None:
            self.bias.model_parallel, self.bias.partition_dim = True, 0

    def forward(self, x_shard):
        return ag_linear(x_shard, self.weight, self.bias, self.group)


class SPRowParallelLinear(nn.Module):
    """Row-parallel linear producing row-sharded output (fused GEMM -> reduce-scatter)."""

    def __init__(self, in_features, out_features, group, bias=True, dtype=torch.bfloat16,
                 device=None, seed=4321, std=0.02):
        super().__init__()
        p, r = group.world, group.rank
        assert in_features % p == 0
        g = torch.Generator().manual_seed(seed)
        full = torch.randn(out_features, in_features, generator=g) * std
        self.group = group
        self.weight = nn.Parameter(full.chunk(p, 1)[r].contiguous().to(dtype).to(device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) \
            if bias else None
        self.weight.model_parallel, self.weight.partition_dim = True, 1

    def forward(self, x, residual=None):
        return linear_rs(x, self.weight, self.bias, residual, self.group)
