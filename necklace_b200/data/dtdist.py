"""Collective helpers for input data (reference: necklace/data/dtdist.py:13-50):
share a shuffled index tensor over the main group, and broadcast a batch (shape
first, then data) from local rank 0 of the tensor-parallel group to its peers.
Shapes travel as int64 (the reference sends them as float32)."""
from __future__ import annotations

import torch

from ..comm import fns, groups


def _is_t(x):
    return isinstance(x, torch.Tensor)


def dt_sampler_do_nccl_bcast(*args, **kw):
    """``(indices, root=0, group=None)``, or the reference's ``(nc, kn, root, buf)`` where
    ``nc`` is a group (or ``None`` = main group) and ``kn`` its size (not needed)."""
    if args and not _is_t(args[0]):
        nc, _kn, root, buf = (list(args) + [None] * 4)[:4]
        buf = kw.get("buf", buf)
        return fns.broadcast(buf, int(kw.get("root", root) or 0), nc or groups.get_nccl_group_main())
    indices = args[0] if args else kw["indices"]
    root = args[1] if len(args) > 1 else kw.get("root", 0)
    group = args[2] if len(args) > 2 else kw.get("group")
    return fns.broadcast(indices, root, group or groups.get_nccl_group_main())


def dt_sampler_do_nccl_allreduce(*args, **kw):
    """``(indices, group=None)``, or the reference's ``(nc, kn, root, buf)``."""
    if args and not _is_t(args[0]):
        nc, buf = args[0], (args[3] if len(args) > 3 else kw.get("buf"))
        return fns.all_reduce(buf, group=nc or groups.get_nccl_group_main())
    indices = args[0] if args else kw["indices"]
    group = args[1] if len(args) > 1 else kw.get("group")
    return fns.all_reduce(indices, group=group or groups.get_nccl_group_main())


def dt_shape_do_nccl_broadcast(a, b=0, group=None):
    """``(shape_tensor, root=0, group=None)``, or the reference's ``(pg, shape_tensor)`` (root
    is rank 0 of the tensor-parallel group there)."""
    if _is_t(a):
        return fns.broadcast(a, b, group or groups.get_nccl_group_mp_or_main())
    return fns.broadcast(b, 0, a or groups.get_nccl_group_mp_or_main())


def dt_input_do_nccl_broadcast(a, b=0, group=None, dtype=None):
    """``(tensor, root=0, group=None)``, or the reference's ``(pg, tensor, dtype='float32')``
    (the tensor carries its type; the name is accepted)."""
    if _is_t(a):
        return fns.broadcast(a, b, group or groups.get_nccl_group_mp_or_main())
    return fns.broadcast(b, 0, a or groups.get_nccl_group_mp_or_main())


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
