"""Megatron ``mpu``-style accessors on top of the group registry
(reference: necklace/frmwrk/pytorch/mpnn/initialize.py:141-200).  Groups come from
``comm.groups``; when a kind is absent the main group stands in, as in the reference."""
from __future__ import annotations

from ....comm import groups as G


def initialize_model_parallel(model_parallel_size_=None):
    """Groups are created by ``init_nccl_groups_map`` / ``init_backend``; nothing to do."""
    return None


def model_parallel_is_initialized():
    return G.get_nccl_group_main() is not None


def get_model_parallel_group():
    return G.get_nccl_group_mp_or_main()


def get_model_parallel_rank():
    g = G.get_nccl_group_mp()
    return g.rank if g is not None else 0


def get_model_parallel_world_size():
    g = G.get_nccl_group_mp()
    return g.world_size if g is not None else 1


def get_model_parallel_src_rank():
    """Global rank of local rank 0 of my tensor-parallel group."""
    g = G.get_nccl_group_mp()
    return g.pg_ranks[0] if g is not None else (G.get_nccl_group_main_rank() or 0)


def get_data_parallel_group():
    return G.get_nccl_group_dp_or_main()


def get_data_parallel_rank():
    g = G.get_nccl_group_dp()
    return g.rank if g is not None else (0 if G.get_nccl_group_mp() else G.get_rank())


def get_data_parallel_world_size():
    g = G.get_nccl_group_dp()
    return g.world_size if g is not None else (1 if G.get_nccl_group_mp() else G.get_world_size())


def destroy_model_parallel():
    G.del_nccl_groups_map_comms()
