"""Group registry under the reference's module name (necklace/cuda/ncclgrp.py)."""
from ..comm.groups import *  # noqa: F401,F403
from ..comm.groups import (GroupInfo as NcclProcessGroup, _S,  # noqa: F401
                           init_nccl_groups_map, get_nccl_groups_map_cfg_dict,
                           get_nccl_groups_map_grp_dict, get_nccl_group_main_grp_list)
