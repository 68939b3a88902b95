"""Collectives on a group: ``all_reduce / all_gather / broadcast / reduce / send / recv``.

Call shapes follow the reference (necklace/cuda/ncclfns.py:32-260): a rank that
is not a member of ``group`` returns at once, the default reduction is a sum, and
``group=None`` means the main group.  Differences: every call is ordered on the
caller's current stream (the reference launches on pynccl's own stream and blocks
on it), tensors living in the symmetric heap take the native peer-memory kernels
(all-reduce, all-gather, broadcast, reduce-scatter), everything else goes through
``torch.distributed`` on the group's process group.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import groups as G

_OPS = {"sum": dist.ReduceOp.SUM, "prod": dist.ReduceOp.PRODUCT, "max": dist.ReduceOp.MAX,
        "min": dist.ReduceOp.MIN}


def _resolve(group):
    group = group or G.get_nccl_group_main()
    return group


def _pg(group):
    """torch.distributed process group handle of a GroupInfo (None = default group)."""
    comm = getattr(group, "comm", None)
    return getattr(comm, "group", None)


def _is_member(group) -> bool:
    return group is None or group.rank >= 0


def _world(group) -> int:
    return 1 if group is None else group.world_size


def _peer(group, t):
    """The PeerGroup of ``group`` if ``t`` lives in its symmetric heap."""
    peer = getattr(getattr(group, "comm", None), "peer", None)
    if peer is None or not t.is_cuda:
        return None
    heap = peer.heap
    off = t.data_ptr() - heap.buf.data_ptr()
    return peer if 0 <= off < heap.nbytes else None


def all_reduce(t: torch.Tensor, op: str = "sum", group=None) -> torch.Tensor:
    group = _resolve(group)
    if not _is_member(group) or _world(group) == 1:
        return t
    peer = _peer(group, t)
    if peer is not None and op == "sum" and t.dtype in (torch.float32, torch.bfloat16) \
            and t.is_contiguous():
        peer.all_reduce(t)
        return t
    dist.all_reduce(t, op=_OPS[op], group=_pg(group))
    return t


def all_gather(out: torch.Tensor, t: torch.Tensor, group=None) -> torch.Tensor:
    """``out`` = concatenation of every member's ``t`` along dim 0 (rank-major)."""
    group = _resolve(group)
    if not _is_member(group):
        return out
    if _world(group) == 1:
        out.view(-1).copy_(t.reshape(-1))
        return out
    peer = _peer(group, out)
    W = _world(group)
    if peer is not None and out.is_contiguous() and out.numel() == W * t.numel() \
            and (out.numel() * out.element_size()) % (16 * W) == 0:
        mine = out.view(-1)[group.rank * t.numel():(group.rank + 1) * t.numel()]
        if mine.data_ptr() != t.data_ptr():
            mine.copy_(t.reshape(-1))
        peer.all_gather(out)          # every member pushes its slice to the others
        return out
    dist.all_gather_into_tensor(out.view(-1), t.contiguous().view(-1), group=_pg(group))
    return out


def broadcast(t: torch.Tensor, root: int = 0, group=None) -> torch.Tensor:
    """``root`` is the rank inside the group."""
    group = _resolve(group)
    if not _is_member(group) or _world(group) == 1:
        return t
    peer = _peer(group, t)
    if peer is not None and t.is_contiguous() and (t.numel() * t.element_size()) % 16 == 0:
        peer.broadcast(t, root)       # the root pushes to every member's copy
        return t
    dist.broadcast(t, src=group.pg_ranks[root], group=_pg(group))
    return t


def reduce(t: torch.Tensor, root: int = 0, op: str = "sum", group=None) -> torch.Tensor:
    group = _resolve(group)
    if not _is_member(group) or _world(group) == 1:
        return t
    dist.reduce(t, dst=group.pg_ranks[root], op=_OPS[op], group=_pg(group))
    return t


def reduce_scatter(out: torch.Tensor, t: torch.Tensor, op: str = "sum", group=None):
    group = _resolve(group)
    if not _is_member(group):
        return out
    if _world(group) == 1:
        out.view(-1).copy_(t.reshape(-1))
        return out
    peer = _peer(group, t)
    W = _world(group)
    if peer is not None and op == "sum" and t.dtype in (torch.float32, torch.bfloat16) \
            and out.dtype == t.dtype and t.is_contiguous() and out.is_contiguous() \
            and t.numel() % (256 * W) == 0 and out.numel() * W == t.numel():
        peer.reduce_scatter(t.view(-1), out.view(-1))
        return out
    dist.reduce_scatter_tensor(out.view(-1), t.contiguous().view(-1), op=_OPS[op],
                               group=_pg(group))
    return out


def send(t: torch.Tensor, dst_global_rank: int):
    """Point-to-point on the main group with global ranks (reference:
    ``do_pp_send_recv``, necklace/frmwrk/pytorch/ptprms.py:417-450)."""
    return dist.isend(t.contiguous(), dst=dst_global_rank)


def recv(t: torch.Tensor, src_global_rank: int):
    return dist.irecv(t, src=src_global_rank)


def barrier(group=None):
    group = _resolve(group)
    if _is_member(group) and _world(group) > 1:
        dist.barrier(group=_pg(group))


# raw-pointer style names of the reference kept as aliases of the tensor forms
pg_all_reduce, pg_all_gather, pg_broadcast, pg_reduce = all_reduce, all_gather, broadcast, reduce
