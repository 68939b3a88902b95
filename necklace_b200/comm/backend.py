"""Communicator bring-up for a worker process.

``init_backend`` plays the part of the reference's unique-id relay and
``ncclCommInitRank`` calls (necklace/trainer/tnopbs.py:407-451, scheduler side
necklace/trainer/tndspp.py:728-751): it joins the ``torch.distributed`` job (NCCL on
GPU, gloo on CPU) whose rendezvous address the scheduler hands out, creates one
process group per dp / pp / mp / zr group of the layout (every rank creates every
group, in the same order) and attaches a communicator object to each of this
rank's ``GroupInfo``.  With ``comm_type='peer'`` it also maps one symmetric
peer-memory heap over all ranks and gives each group a ``PeerGroup`` view for the
fused kernels; there are no fixed sleeps.
"""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist

from . import groups as G
from .symm import PeerGroup, SymmetricHeap, TorchGroup

_STATE = {"heap": None, "inited_here": False}


class GroupComm(TorchGroup):
    """A ``TorchGroup`` plus (optionally) the peer-memory view of the same ranks."""

    def __init__(self, pg, ranks, my_global_rank, peer: PeerGroup | None = None):
        self.group = pg
        self.ranks = list(ranks)
        self.world = len(ranks)
        self.rank = self.ranks.index(my_global_rank) if my_global_rank in self.ranks else -1
        self.member = self.rank >= 0
        self.peer = peer


def init_backend(tmode: str, cfg: dict, comm_type: str = "nccl", device=None,
                 master_addr: str = "127.0.0.1", master_port: int = 29400,
                 heap_bytes: int = 0, timeout_s: float = 120.0):
    """Returns the symmetric heap (or None).  ``cfg`` is the group cfg dict
    (``world_size, my_rank, dp_size, ...``)."""
    world, rank = cfg["world_size"], cfg["my_rank"]
    G.init_nccl_groups_map(tmode, cfg)
    use_cuda = device is not None and torch.device(device).type == "cuda"
    backend = "gloo" if (comm_type == "gloo" or not use_cuda) else "nccl"
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", master_addr)
        os.environ.setdefault("MASTER_PORT", str(master_port))
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device(device)
        dist.init_process_group(backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
        _STATE["inited_here"] = True
    heap = None
    if comm_type == "peer" and use_cuda and heap_bytes > 0:
        heap = SymmetricHeap(heap_bytes, device=device)
        _STATE["heap"] = heap
    main = G.get_nccl_group_main()
    main.attach_comm(GroupComm(None, main.pg_ranks, rank,
                               heap.peer_group(main.pg_ranks) if heap else None))
    mine = G.get_nccl_groups_map()
    for key, all_groups in G.get_nccl_groups_map_grp_dict().items():
        for ranks in all_groups:
            pg = dist.new_group(ranks) if world > 1 and len(ranks) > 1 else None
            peer = heap.peer_group(ranks) if heap else None
            if rank in ranks and key in mine:
                mine[key].attach_comm(GroupComm(pg, ranks, rank, peer))
    if world > 1 and "pp_group" in G.get_nccl_groups_map_grp_dict():
        from ..parallel.pipeline import create_channels
        create_channels(G.get_nccl_groups_map_grp_dict()["pp_group"])
    return heap


def get_heap():
    return _STATE["heap"]


def shutdown_backend():
    G.del_nccl_groups_map_comms()
    _STATE["heap"] = None
    if dist.is_initialized() and _STATE["inited_here"]:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass
    _STATE["inited_here"] = False
