"""The older two-way (data x model parallel) group map under the reference's module name
(necklace/cuda/ncclpgs.py:19-337; superseded there by ``ncclgrp`` and kept for scripts that
still import it).  Layout as in the reference: model-parallel groups are runs of adjacent
ranks, data-parallel groups stride over them (8 ranks, mp 2: mp [0,1] [2,3] [4,5] [6,7];
dp [0,2,4,6] [1,3,5,7]).  Everything is served by ``comm.groups``."""
from __future__ import annotations

from ..comm import groups as _G
from ..comm.groups import (GroupInfo as NcclProcessGroup, del_nccl_groups_map_comms, divide,  # noqa: F401
                           ensure_divisibility, get_nccl_group_dp, get_nccl_group_dp_or_main,
                           get_nccl_group_main, get_nccl_group_main_rank,
                           get_nccl_group_main_world_size, get_nccl_group_mp,
                           get_nccl_group_mp_or_main, get_nccl_groups_map,
                           get_nccl_groups_map_cfg_dict, get_nccl_groups_map_grp_dict, get_rank,
                           get_world_size, get_nccl_main_nk, make_pg_by_nc, make_pg_by_nk,
                           set_nccl_group_main_by_nc, set_nccl_group_main_rank,
                           set_nccl_group_main_world_size, set_nccl_groups_map)


build_pg_cfg = _G.build_pg_cfg


def init_nccl_groups_map(world_size, my_rank, mp_size, dp_size=None, is_worker=True):
    """Main group plus this rank's data- and model-parallel groups."""
    mp = min(int(mp_size), int(world_size))
    ensure_divisibility(world_size, mp)
    dp = divide(world_size, mp)
    if dp_size not in (None, 0, dp):
        raise ValueError(f"dp_size {dp_size} * mp_size {mp} != world_size {world_size}")
    _G.init_nccl_groups_map("dp+mp", {"world_size": world_size, "my_rank": my_rank,
                                      "dp_size": dp, "mp_size": mp, "is_worker": is_worker})
