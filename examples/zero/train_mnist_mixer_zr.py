"""ZeRO (``zr`` / ``dp+zr``) training of an MLP-Mixer on MNIST-shaped data, the layer-owner
way of the reference: ``net_map`` unit i is owned by zr rank i, its weights are broadcast
before its forward, its gradients reduced to the owner after its backward, only the owner
keeps an optimizer for it (reference: examples/zero/mnist/pytorch/train_mnist_zr_2_mlpmx.py,
train_mnist_zf_2.py for ``--flat``, train_mnist_zr_5_dpzr_2.py for ``dp+zr``).

    python train_mnist_mixer_zr.py -r scheduler -w 3 -u ipc:///tmp/s.ipc -e 1
    python train_mnist_mixer_zr.py -r worker -w 3 -k <r> -u ipc:///tmp/w<r>.ipc -s ipc:///tmp/s.ipc \
        [-t zr] [--flat] [--offload] [--stepwise] [--no-cuda]

An after-epoch hook evaluates the re-assembled whole network on rank 0
(``trnr.get_whole_net_cpu()``), as the reference's ZeRO examples do."""
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
from necklace_b200.data.dtldngn import DataLoaderNgnBase
from necklace_b200.data.dtset import SyntheticDataset
from necklace_b200.data.sampler import SliceSampler
from necklace_b200.models.mlp_mixer import mixer_parts
from necklace_b200.trainer import tndszd
from necklace_b200.trainer.zroppd import TrainerMPOPPytorch
from necklace_b200.trainer.zroppf import TrainerMPOPPytorch as FlatTrainer
from necklace_b200.utils.argutils import attach_nk_args_parser, pg_cfg_from_args
from necklace_b200.utils.hookbase import NklcHookBase


class HookEvalWholeNet(NklcHookBase):
    def __init__(self, net, ctx, ds, out):
        super().__init__(net, ctx)
        self.ds, self.out, self.acc = ds, out, []

    def __call__(self, trnr, *args, **kwargs):
        whole = trnr.get_whole_net_cpu().eval()
        x = torch.stack([self.ds[j][0] for j in range(64)])
        y = torch.tensor([self.ds[j][1] for j in range(64)])
        with torch.no_grad():
            out = whole(x.float())
            out = out[0] if isinstance(out, (tuple, list)) else out
        self.acc.append(float((out.argmax(1) == y).float().mean()))
        print(f"[{trnr.ti}] epoch {trnr.e} train-subset accuracy {self.acc[-1]:.3f}", flush=True)


def main():
    ap = argparse.ArgumentParser()
    attach_nk_args_parser(ap)
    ap.add_argument("--batch-size", "-b", type=int, default=32)
    ap.add_argument("--lr", type=float, default=0.05)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--no-cuda", action="store_true")
    ap.add_argument("--dataset-len", type=int, default=256)
    ap.add_argument("--parts", type=int, default=0)
    ap.add_argument("--flat", action="store_true", help="flat-buffer flavour (zroppf)")
    ap.add_argument("--offload", action="store_true")
    ap.add_argument("--stepwise", action="store_true")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    tmode = args.tmode or "zr"
    pg_cfg = pg_cfg_from_args(args)
    ncclgrp.init_nccl_groups_map(tmode, pg_cfg)
    grp_map = ncclgrp.get_nccl_groups_map_grp_dict()
    zr_size = len(grp_map["zr_group"][0])
    n_parts = args.parts or max(zr_size, 2)
    typ = "dpzr" if tmode == "dp+zr" else "oozr"

    if args.role == "scheduler":
        net_map = OrderedDict((i, {"net_map_order": i}) for i in range(n_parts))
        svc = tndszd.MPSVCScheduler({"url": args.url, "workers": args.world_size,
                                     "epochs": args.epochs, "nccl_allreduce_typ": typ,
                                     "stepwise": args.stepwise, "net_map": net_map,
                                     "nccl_groups_grp_map": grp_map, "phase_timeout": 120})
        svc.loop()
        print("scheduler:", svc.exit_status)
        return 0 if svc.exit_status == "finished" else 1

    use_cuda = torch.cuda.is_available() and not args.no_cuda
    necklace_b200.init(args.gpu_rank)
    ctx = torch.device("cuda", int(args.gpu_rank)) if use_cuda else torch.device("cpu")
    parts = mixer_parts(n_parts, seed=args.seed)
    net_map = OrderedDict((i, {"net": p, "net_map_order": i}) for i, p in enumerate(parts))
    ds = SyntheticDataset(args.dataset_len, (1, 28, 28), classes=10, seed=args.seed)

    def dataloader_creator():
        per = len(ds) // args.world_size
        sampler = SliceSampler(indices=list(range(args.rank * per, (args.rank + 1) * per)))
        return DataLoaderNgnBase(ds, batch_size=args.batch_size, sampler=sampler,
                                 last_batch="discard")

    trainer_cfg = {
        "kn": args.world_size, "ti": args.rank, "ctx": ctx, "loss": nn.CrossEntropyLoss(),
        "batch_size": args.batch_size, "epochs": args.epochs, "dataset_len": args.dataset_len,
        "dataloader_type": "dp", "dataloader_creator": dataloader_creator, "log_interval": 0,
        "tmode": tmode, "pg_cfg": pg_cfg, "comm_type": "gloo" if not use_cuda else args.comm_type,
        "net_map": net_map, "net_map_maxlen": n_parts,
        "optimizer_creator": lambda net: torch.optim.SGD(net.parameters(), lr=args.lr),
        "offload": args.offload, "zr_grad_average": True,
    }
    svc = tndszd.MPSVCWorker({"url": args.url, "scheduler_url": args.server_url,
                              "rank": args.rank,
                              "trainer_cls": FlatTrainer if args.flat else TrainerMPOPPytorch,
                              "trainer_cfg": trainer_cfg})
    hook = HookEvalWholeNet(None, ctx, ds, args.out)
    if args.rank == 0:
        svc.svr.trnr.register_hook_after_epoch(hook)
    svc.loop()
    trnr = svc.svr.trnr
    if args.out:
        w = float(sum(p.detach().double().sum() for m in trnr.nets for p in m.parameters()))
        json.dump({"rank": args.rank, "status": svc.exit_status, "weights_sum": w,
                   "loss": float(trnr.last_loss) if trnr.last_loss is not None else None,
                   "acc": hook.acc}, open(args.out, "w"))
    print(f"worker {args.rank}:", svc.exit_status)
    return 0 if svc.exit_status == "stopped" else 1


if __name__ == "__main__":
    sys.exit(main())
