"""One script for every trainer mode on a small MLP: ``dp``, ``mp``, ``dp+mp``, ``pp``, ``dp+pp``,
``dp+pp+mp``, ``zr``, ``dp+zr``, ``zr+mp``, ``dp+zr+mp``.

It plays the role of the reference's per-mode MNIST examples (examples/mp/.../
train_mnist_mpnn_22_mpdp_grps.py, examples/pp/.../train_mnist_pp_81_dpppmp_3.py,
examples/zero/.../train_mnist_zr_8_dpzrmp_3.py) with synthetic 784-feature inputs:

    python train_mlp_hybrid.py -r scheduler -w 4 -t dp+pp -dpsz 2 -ppsz 2 -u ipc:///tmp/s.ipc
    python train_mlp_hybrid.py -r worker -w 4 -k <r> -t dp+pp -dpsz 2 -ppsz 2 \
        -u ipc:///tmp/w<r>.ipc -s ipc:///tmp/s.ipc [--no-cuda]

The network is cut into ``net_map`` units; with ``mp`` in the mode the hidden layers are
``ColumnParallelLinear`` / ``RowParallelLinear`` pairs.  At the end every worker writes its
last loss and a weight checksum to ``--out``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from collections import OrderedDict

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch
import torch.nn as nn

import necklace_b200
from necklace_b200.comm import groups as ncclgrp
from necklace_b200.data.dtdummy import DtldDummy, DtstDummy
from necklace_b200.data.dtldngn import DataLoaderNgnBase
from necklace_b200.data.dtset import SyntheticDataset
from necklace_b200.data.sampler import SliceSampler
from necklace_b200.frmwrk.pytorch import mpnn
from necklace_b200.trainer import service
from necklace_b200.utils.argutils import attach_nk_args_parser, pg_cfg_from_args

HID = 64


class MpBlock(nn.Module):
    """Column-parallel up projection, ReLU, row-parallel down projection."""

    def __init__(self, d_in, d_hid, d_out, seed):
        super().__init__()
        self.up = mpnn.ColumnParallelLinear(d_in, d_hid, gather_output=False, seed=seed)
        self.down = mpnn.RowParallelLinear(d_hid, d_out, input_is_parallel=True, seed=seed + 1)

    def forward(self, x):
        return self.down(torch.relu(self.up(x)))


def build_parts(n_parts, use_mp, seed):
    torch.manual_seed(seed)
    dims = [784] + [HID] * (n_parts - 1) + [10]
    parts = []
    for i in range(n_parts):
        if use_mp:
            blk = MpBlock(dims[i], 2 * HID, dims[i + 1], seed=seed + 10 * i)
        else:
            blk = nn.Sequential(nn.Linear(dims[i], 2 * HID), nn.ReLU(), nn.Linear(2 * HID, dims[i + 1]))
        parts.append(blk if i == n_parts - 1 else nn.Sequential(blk, nn.ReLU()))
    return parts


def main(build=None, in_shape=(784,)):
    """``build(n_parts, use_mp, seed)`` returns the ``net_map`` units (default: the MLP of this
    file) for inputs of shape ``in_shape``; other examples reuse this driver with their own
    network (examples/pp/train_mnist_pp.py, examples/mp/train_mnist_mpnn.py)."""
    build = build or build_parts
    ap = argparse.ArgumentParser()
    attach_nk_args_parser(ap)
    ap.add_argument("--batch-size", "-b", type=int, default=32)
    ap.add_argument("--lr", type=float, default=0.05)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--no-cuda", action="store_true")
    ap.add_argument("--dataset-len", type=int, default=256)
    ap.add_argument("--stepwise", action="store_true")
    ap.add_argument("--micro-batches", type=int, default=1)
    ap.add_argument("--parts", type=int, default=0, help="number of net_map units")
    ap.add_argument("--zr-flat", action="store_true")
    ap.add_argument("--zr-offload", action="store_true")
    ap.add_argument("--out", type=str, default="")
    args = ap.parse_args()

    tmode = args.tmode or "dp"
    kinds = tmode.split("+")
    pg_cfg = pg_cfg_from_args(args)
    ncclgrp.init_nccl_groups_map(tmode, pg_cfg)
    grp_map = ncclgrp.get_nccl_groups_map_grp_dict()
    size = lambda k: len(grp_map[k + "_group"][0]) if k + "_group" in grp_map else 1
    n_parts = args.parts or (size("pp") if "pp" in kinds else (3 if "zr" in kinds else 1))
    typ = {"zr": "oozr", "dp+zr": "dpzr", "zr+mp": "zrmp", "dp+zr+mp": "dpzrmp",
           "mp": "oopt"}.get(tmode, "grad")

    if args.role == "scheduler":
        net_map = OrderedDict((i, {"net_map_order": i}) for i in range(n_parts))
        if "pp" in kinds:
            for i in range(n_parts):
                net_map[i]["worker_rank"] = grp_map["pp_group"][0][i]
        svc = service.SVCScheduler({
            "url": args.url, "workers": args.world_size, "epochs": args.epochs,
            "nccl_allreduce_typ": typ, "stepwise": args.stepwise, "net_map": net_map,
            "nccl_groups_grp_map": grp_map, "phase_timeout": 120})
        svc.loop()
        print("scheduler:", svc.exit_status)
        return 0 if svc.exit_status == "finished" else 1

    use_cuda = torch.cuda.is_available() and not args.no_cuda
    necklace_b200.init(args.gpu_rank)
    ctx = torch.device("cuda", int(args.gpu_rank)) if use_cuda else torch.device("cpu")
    parts = build(n_parts, "mp" in kinds, args.seed)
    net_map = OrderedDict((i, {"net": p, "net_map_order": i}) for i, p in enumerate(parts))

    # which data replica am I?  ranks that differ only in pp / mp coordinates share data
    def coord(kind):
        g = ncclgrp.get_nccl_groups_map().get(kind + "_group")
        return g.rank if g is not None else 0
    replica = coord("dp") * size("zr") + coord("zr")
    n_replica = size("dp") * size("zr")
    mp_rank = coord("mp")

    def dataloader_creator():
        ds = SyntheticDataset(args.dataset_len, tuple(in_shape), classes=10, seed=args.seed)
        per = len(ds) // n_replica
        if "mp" in kinds and mp_rank != 0:
            return DtldDummy(DtstDummy(per), args.batch_size)
        sampler = SliceSampler(indices=list(range(replica * per, (replica + 1) * per)))
        return DataLoaderNgnBase(ds, batch_size=args.batch_size, sampler=sampler,
                                 last_batch="discard")

    trainer_cfg = {
        "kn": args.world_size, "ti": args.rank, "ctx": ctx, "loss": nn.CrossEntropyLoss(),
        "batch_size": args.batch_size, "epochs": args.epochs, "dataset_len": args.dataset_len,
        "dataloader_type": "mpdp" if "mp" in kinds else "dp",
        "dataloader_data_shape_dims": [len(in_shape) + 1, 1],
        "dataloader_creator": dataloader_creator,
        "log_interval": 0, "tmode": tmode, "pg_cfg": pg_cfg,
        "comm_type": "gloo" if not use_cuda else args.comm_type,
        "net_map": net_map, "net_map_maxlen": n_parts, "micro_batches": args.micro_batches,
    }
    if "zr" in kinds:
        from necklace_b200.trainer.zroppd import TrainerMPOPPytorch as Trainer
        trainer_cfg.update(optimizer_creator=lambda net: torch.optim.SGD(net.parameters(), lr=args.lr),
                           flat=args.zr_flat, offload=args.zr_offload, zr_grad_average=True)
    elif "pp" in kinds:
        from necklace_b200.trainer.ppoppt import TrainerMPOPPytorch as Trainer
        stage = coord("pp")
        trainer_cfg.update(net_map_order=stage, net=parts[stage],
                           opt=torch.optim.SGD(parts[stage].parameters(), lr=args.lr))
    else:
        from necklace_b200.trainer.tnoppt import TrainerOPPytorch as Trainer
        net = nn.Sequential(*parts)
        trainer_cfg.update(net=net, opt=torch.optim.SGD(net.parameters(), lr=args.lr))
    svc = service.SVCWorker({"url": args.url, "scheduler_url": args.server_url, "rank": args.rank,
                             "trainer_cls": Trainer, "trainer_cfg": trainer_cfg})
    svc.loop()
    trnr = svc.svr.trnr
    if args.out:
        if "zr" in kinds:
            mods = [p for p in trnr.nets]
        else:
            mods = [trnr.net]
        w = {f"{mi}.{n}": float(p.detach().double().sum()) for mi, m in enumerate(mods)
             for n, p in m.named_parameters()}
        with open(args.out, "w") as f:
            json.dump({"rank": args.rank, "status": svc.exit_status, "steps": trnr.i,
                       "loss": float(trnr.last_loss) if trnr.last_loss is not None else None,
                       "weights": w}, f)
    print(f"worker {args.rank}:", svc.exit_status)
    return 0 if svc.exit_status == "stopped" else 1


if __name__ == "__main__":
    sys.exit(main())
