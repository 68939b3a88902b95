"""The framework command line (role / world / rank / gpu / trainer mode / group sizes).

Flag names, short forms and defaults are those of the reference CLI
(necklace/utils/argutils.py:6-55) so launch scripts carry over; ``--comm_type``
gains the value ``peer`` (NVLink peer-memory collectives, the default on GPU) next
to ``nccl`` (torch.distributed NCCL baseline path) and ``gloo`` (CPU).
"""
from __future__ import annotations

import os

from . import osutils


def attach_nk_args_parser(parser):
    a = parser.add_argument
    a("--epochs", "-e", type=int, default=10, help="number of epochs to train")
    a("--gpu_rank", "-g", default="0", type=str, help="GPU device to train with")
    a("--url", "-u", type=str, default="ipc:///tmp/nk-wkr-1.ipc", help="this node's RPC url")
    a("--server-url", "-s", type=str, default="ipc:///tmp/nk-svr-1.ipc", help="scheduler url")
    a("--role", "-r", type=str, default="worker", help="scheduler or worker")
    a("--world-size", "-w", type=int, default=1, help="number of workers")
    a("--rank", "-k", type=int, default=0, help="global rank of this worker")
    a("--local_rank", "-lk", type=int, default=-1, help="local rank (unused, kept for launchers)")
    a("--rpc_ifname", "-ri", type=str, default="", help="NIC whose address the RPC url uses")
    a("--rpc_ip_prefix", "-rp", type=str, default="", help="address prefix the RPC url uses")
    a("--comm_ifname", "-ci", type=str, default="", help="NIC for the collective bootstrap")
    a("--comm_type", "-x", type=str, default="nccl", help="nccl | peer | gloo")
    a("--tmode", "-t", type=str, default="", help="trainer mode, e.g. dp+pp+mp")
    a("--dp-size", "-dpsz", type=int, default=0, help="data-parallel group size")
    a("--mp-size", "-mpsz", type=int, default=0, help="tensor-parallel group size")
    a("--pp-size", "-ppsz", type=int, default=0, help="pipeline-parallel group size")
    a("--zr-size", "-zrsz", type=int, default=0, help="ZeRO group size")
    return parser


def args_remake(args, **kwargs):
    """Post-launcher fix-up (reference: argutils.py:58-92): derive the local GPU index
    from ``rank % nslot`` and expand ``@{MY_IP}``, ``@{LOCAL_RANK}`` and ``@{RANK}``
    in ``--url``."""
    nslot = int(getattr(args, "nslot", 0) or kwargs.get("nslot", 0) or 1)
    local_rank = args.rank % nslot
    args.gpu_dev_i = local_rank
    if args.rpc_ifname:
        my_ip = osutils.get_ip_by_nic(args.rpc_ifname)
    elif args.rpc_ip_prefix:
        my_ip = osutils.get_ip_by_prefix(args.rpc_ip_prefix)
    else:
        my_ip = osutils.get_ip_by_first()
    args.url = (args.url.replace("@{MY_IP}", my_ip or "127.0.0.1")
                .replace("@{LOCAL_RANK}", str(local_rank)).replace("@{RANK}", str(args.rank)))
    if args.comm_ifname:
        os.environ.setdefault("NCCL_SOCKET_IFNAME", args.comm_ifname)
        os.environ.setdefault("GLOO_SOCKET_IFNAME", args.comm_ifname)
    return args


def pg_cfg_from_args(args) -> dict:
    """The cfg dict ``init_nccl_groups_map`` expects, from parsed CLI flags."""
    return {"world_size": args.world_size, "my_rank": args.rank, "dp_size": args.dp_size,
            "pp_size": args.pp_size, "mp_size": args.mp_size, "zr_size": args.zr_size,
            "is_worker": args.role == "worker"}
