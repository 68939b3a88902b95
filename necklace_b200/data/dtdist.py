"""Collective helpers for input data (reference: necklace/data/dtdist.py:13-50):
share a shuffled index tensor over the main group, and broadcast a batch (shape
first, then data) from local rank 0 of the tensor-parallel group to its peers.
Shapes travel as int64 (the reference sends them as float32)."""
from __future__ import annotations

import torch

from ..comm import fns, groups


def dt_sampler_do_nccl_bcast(indices: torch.Tensor, root: int = 0, group=None):
    return fns.broadcast(indices, root, group or groups.get_nccl_group_main())


def dt_sampler_do_nccl_allreduce(indices: torch.Tensor, group=None):
    return fns.all_reduce(indices, group=group or groups.get_nccl_group_main())


def dt_shape_do_nccl_broadcast(shape_t: torch.Tensor, root: int = 0, group=None):
    return fns.broadcast(shape_t, root, group or groups.get_nccl_group_mp_or_main())


def dt_input_do_nccl_broadcast(t: torch.Tensor, root: int = 0, group=None):
    return fns.broadcast(t, root, group or groups.get_nccl_group_mp_or_main())


def broadcast_batch(tensors, ndims, dtypes, device, root: int = 0, group=None):
    """Rank ``root`` of the group passes its tensors; the others pass ``None`` and get
    freshly allocated copies.  ``ndims`` / ``dtypes`` describe every tensor so the
    receivers know how many shape entries to expect."""
    group = group or groups.get_nccl_group_mp_or_main()
    out = []
    is_root = group.rank == root
    for i, (nd, dt) in enumerate(zip(ndims, dtypes)):
        shp = torch.zeros(nd, dtype=torch.int64, device=device)
        if is_root:
            shp.copy_(torch.tensor(list(tensors[i].shape), dtype=torch.int64))
        dt_shape_do_nccl_broadcast(shp, root, group)
        if is_root:
            t = tensors[i].to(device=device, dtype=dt).contiguous()
        else:
            t = torch.empty([int(x) for x in shp.tolist()], dtype=dt, device=device)
        dt_input_do_nccl_broadcast(t, root, group)
        out.append(t)
    return out
