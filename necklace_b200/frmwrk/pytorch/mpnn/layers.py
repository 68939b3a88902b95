"""Tensor-parallel layers (Megatron style) on the native GEMM.

``ColumnParallelLinear`` keeps ``[out/p, in]`` of the weight, ``RowParallelLinear``
``[out, in/p]``, ``VocabParallelEmbedding`` a contiguous slice of the vocabulary and
``ParallelEmbedding`` a slice of the embedding dimension; all mark their weights
``model_parallel = True`` (reference: necklace/frmwrk/pytorch/mpnn/layers.py:40-328).
Weights are initialised from one master weight that every rank generates with the
same seed and then slices, so the assembled layer equals its single-GPU counterpart.
Matmuls run on the tcgen05 GEMM (``ops.linear``) for bf16 CUDA tensors.  When the
tensor-parallel group has a peer-memory view (communicator brought up with
``comm_type='peer'``) the all-reduce of ``RowParallelLinear``'s output and of
``ColumnParallelLinear``'s input gradient is not an NCCL call after the GEMM but the fused
GEMM -> reduce-scatter kernel followed by the peer-memory all-gather
(``parallel.tensor.RowLinearFn`` / ``ColumnLinearFn``); set ``NKB_TP_FUSED=0`` to force the
NCCL path (the baseline).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ....ops import linear as nk_linear
from . import initialize as mpu
from .mappings import (copy_to_model_parallel_region, gather_from_model_parallel_region,
                       reduce_from_model_parallel_region, scatter_to_model_parallel_region)
from .utils import VocabUtility, divide


def _initialize_affine_weight(weight, out_features, in_features, per_partition_size,
                              partition_dim, init_method, stride=1, return_master_weight=False,
                              seed=None):
    """Build the full weight (CPU, fp32), keep my slice(s) along ``partition_dim``."""
    weight.model_parallel = True
    weight.partition_dim = partition_dim
    weight.partition_stride = stride
    ws, rank = mpu.get_model_parallel_world_size(), mpu.get_model_parallel_rank()
    gen_state = torch.random.get_rng_state() if seed is not None else None
    if seed is not None:
        torch.manual_seed(seed)
    master = torch.empty(out_features, in_features, dtype=torch.float32)
    init_method(master)
    if gen_state is not None:
        torch.random.set_rng_state(gen_state)
    if ws == 1:
        with torch.no_grad():
            weight.copy_(master.to(weight.dtype))
        return master if return_master_weight else None
    per_stride = divide(per_partition_size, stride)
    pieces = torch.split(master, per_stride, dim=partition_dim)
    mine = pieces[rank::ws]
    with torch.no_grad():
        weight.copy_(torch.cat(mine, dim=partition_dim).to(weight.dtype))
    return master if return_master_weight else None


def _linear(x, w, b=None):
    if x.is_cuda and x.dtype == torch.bfloat16:
        return nk_linear(x, w, b)
    return F.linear(x, w, b)


def _fused_group(x):
    """PeerGroup for the fused kernels, or None (see ``parallel.tensor.fused_group_of``)."""
    import os
    if os.environ.get("NKB_TP_FUSED", "1") == "0":
        return None
    from ....comm import groups as G
    from ....parallel.tensor import fused_group_of
    g = G.get_nccl_group_mp()
    if g is None or g.world_size == 1:
        return None
    return fused_group_of(g, x, x.numel() // x.shape[-1])


class VocabParallelEmbedding(nn.Module):
    def __init__(self, num_embeddings, embedding_dim, padding_idx=None,
                 init_method=nn.init.xavier_normal_, dtype=torch.float32, device=None,
                 seed=1234):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.padding_idx = padding_idx
        ws = mpu.get_model_parallel_world_size()
        self.vocab_start_index, self.vocab_end_index = \
            VocabUtility.vocab_range_from_global_vocab_size(num_embeddings,
                                                            mpu.get_model_parallel_rank(), ws)
        self.num_embeddings_per_partition = self.vocab_end_index - self.vocab_start_index
        self.weight = nn.Parameter(torch.empty(self.num_embeddings_per_partition, embedding_dim,
                                               dtype=dtype, device=device))
        _initialize_affine_weight(self.weight, num_embeddings, embedding_dim,
                                  self.num_embeddings_per_partition, 0, init_method, seed=seed)

    def forward(self, input_):
        mask = (input_ < self.vocab_start_index) | (input_ >= self.vocab_end_index)
        local = (input_ - self.vocab_start_index).masked_fill(mask, 0)
        out = F.embedding(local, self.weight, self.padding_idx)
        out = out.masked_fill(mask.unsqueeze(-1), 0.0)
        return reduce_from_model_parallel_region(out)


class ParallelEmbedding(nn.Module):
    def __init__(self, num_embeddings, embedding_dim, padding_idx=None,
                 init_method=nn.init.xavier_normal_, keep_master_weight_for_test=False,
                 dtype=torch.float32, device=None, seed=1234):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.padding_idx = padding_idx
        ws = mpu.get_model_parallel_world_size()
        self.embedding_dim_per_partition = divide(embedding_dim, ws)
        self.weight = nn.Parameter(torch.empty(num_embeddings, self.embedding_dim_per_partition,
                                               dtype=dtype, device=device))
        _initialize_affine_weight(self.weight, num_embeddings, embedding_dim,
                                  self.embedding_dim_per_partition, 1, init_method, seed=seed)

    def forward(self, input_):
        input_parallel = copy_to_model_parallel_region(input_) if input_.is_floating_point() \
            else input_
        out = F.embedding(input_parallel, self.weight, self.padding_idx)
        return gather_from_model_parallel_region(out)


class ColumnParallelLinear(nn.Module):
    """``Y = X A^T + b`` with ``A`` split along its output dimension."""

    def __init__(self, in_features, out_features, bias=True, gather_output=True,
                 init_method=nn.init.xavier_normal_, stride=1, keep_master_weight_for_test=False,
                 dtype=torch.float32, device=None, seed=1234):
        super().__init__()
        self.in_features, self.out_features, self.gather_output = in_features, out_features, \
            gather_output
        ws = mpu.get_model_parallel_world_size()
        self.output_size_per_partition = divide(out_features, ws)
        self.weight = nn.Parameter(torch.empty(self.output_size_per_partition, in_features,
                                               dtype=dtype, device=device))
        if bias:
            self.bias = nn.Parameter(torch.zeros(self.output_size_per_partition, dtype=dtype,
                                                 device=device))
            self.bias.model_parallel = True
            self.bias.partition_dim = 0
        else:
            self.register_parameter("bias", None)
        self.master_weight = _initialize_affine_weight(
            self.weight, out_features, in_features, self.output_size_per_partition, 0,
            init_method, stride=stride, return_master_weight=keep_master_weight_for_test,
            seed=seed)

    def forward(self, input_):
        peer = _fused_group(input_)
        if peer is not None:
            from ....parallel.tensor import ColumnLinearFn
            x2 = input_.reshape(-1, input_.shape[-1])
            out = ColumnLinearFn.apply(x2, self.weight, self.bias, peer)
            out = out.view(*input_.shape[:-1], out.shape[-1])
        else:
            input_parallel = copy_to_model_parallel_region(input_)
            out = _linear(input_parallel, self.weight, self.bias)
        return gather_from_model_parallel_region(out) if self.gather_output else out


class RowParallelLinear(nn.Module):
    """``Y = X A^T + b`` with ``A`` split along its input dimension; partial results are
    all-reduced and the bias is added once, after the reduction."""

    def __init__(self, in_features, out_features, bias=True, input_is_parallel=False,
                 init_method=nn.init.xavier_normal_, stride=1, keep_master_weight_for_test=False,
                 dtype=torch.float32, device=None, seed=1234):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.input_is_parallel = input_is_parallel
        ws = mpu.get_model_parallel_world_size()
        self.input_size_per_partition = divide(in_features, ws)
        self.weight = nn.Parameter(torch.empty(out_features, self.input_size_per_partition,
                                               dtype=dtype, device=device))
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device))
        else:
            self.register_parameter("bias", None)
        self.master_weight = _initialize_affine_weight(
            self.weight, out_features, in_features, self.input_size_per_partition, 1,
            init_method, stride=stride, return_master_weight=keep_master_weight_for_test,
            seed=seed)

    def forward(self, input_):
        input_parallel = input_ if self.input_is_parallel else \
            scatter_to_model_parallel_region(input_)
        peer = _fused_group(input_parallel)
        if peer is not None:
            from ....parallel.tensor import RowLinearFn
            x2 = input_parallel.reshape(-1, input_parallel.shape[-1])
            out = RowLinearFn.apply(x2, self.weight, peer)
            out = out.view(*input_parallel.shape[:-1], out.shape[-1])
        else:
            out = reduce_from_model_parallel_region(_linear(input_parallel, self.weight))
        return out + self.bias if self.bias is not None else out
