"""Data-parallel (or single-worker) LeNet on MNIST-shaped data: the canonical example.

Start one scheduler and N workers from this same script, as with the reference
(examples/dp/mnist/pytorch/train_ngn_mnist_1.py:216-307):

    python train_mnist_dp.py -r scheduler -w 2 -u ipc:///tmp/nk-svr.ipc -e 1
    python train_mnist_dp.py -r worker -w 2 -k 0 -u ipc:///tmp/nk-w0.ipc -s ipc:///tmp/nk-svr.ipc -t dp
    python train_mnist_dp.py -r worker -w 2 -k 1 -u ipc:///tmp/nk-w1.ipc -s ipc:///tmp/nk-svr.ipc -t dp

``--loader shm|queue|obj`` feeds the workers from loader processes through shared memory
(the reference's train_ngn_mnist_2_dtpt.py; loaders in dtloader.py).  Data is synthetic (uniform
[0,1) images, uniform labels) unless ``--data-dir`` points at torchvision MNIST files.  ``--no-cuda`` keeps everything on the CPU (gloo collectives).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch
import torch.nn as nn

import necklace_b200
from necklace_b200.comm import groups as ncclgrp
from necklace_b200.data.dtldngn import DataLoaderNgnBase
from necklace_b200.data.dtset import SyntheticDataset
from necklace_b200.data.sampler import SliceSampler
from necklace_b200.models.lenet import LeNet
from necklace_b200.trainer import tndsnc
from necklace_b200.trainer.tnoppt import TrainerOPPytorch
from necklace_b200.utils.argutils import attach_nk_args_parser, pg_cfg_from_args
from necklace_b200.utils.hookbase import NklcHookBase
from necklace_b200.utils.wrpbase import NklcWrapperBase


class WrpDoLoss(NklcWrapperBase):
    def __init__(self, net, ctx):
        super().__init__(net, ctx)
        self.ce = nn.CrossEntropyLoss()

    def __call__(self, output, target):
        return self.ce(output, target)


class HookLogLoss(NklcHookBase):
    """After every epoch: append the mean training loss and the host seconds of the epoch to
    a JSON file."""

    def __init__(self, net, ctx, path):
        super().__init__(net, ctx)
        self.path, self.losses, self.epochs = path, [], []
        self.seconds, self.steps, self.t0 = [], [], None

    def on_batch(self, trnr, ret=None):
        if self.t0 is None:
            self.t0 = time.time()             # the epoch's clock starts after its first step
        if trnr.last_loss is not None and ret == "one_step":
            self.losses.append(float(trnr.last_loss))

    def __call__(self, trnr, *args, **kwargs):
        self.epochs.append(sum(self.losses) / max(len(self.losses), 1))
        self.seconds.append(time.time() - (self.t0 or time.time()))
        self.steps.append(max(len(self.losses) - 1, 0))
        self.losses, self.t0 = [], None
        if self.path:
            with open(self.path, "w") as f:
                json.dump({"rank": trnr.ti, "epoch_loss": self.epochs,
                           "epoch_seconds": self.seconds, "epoch_steps": self.steps,
                           "weights_sum": float(sum(p.double().sum() for p in
                                                    trnr.net.parameters()))}, f)


def main():
    ap = argparse.ArgumentParser()
    attach_nk_args_parser(ap)
    ap.add_argument("--batch-size", "-b", type=int, default=100)
    ap.add_argument("--lr", type=float, default=0.01)
    ap.add_argument("--momentum", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--log-interval", type=int, default=100)
    ap.add_argument("--no-cuda", action="store_true")
    ap.add_argument("--dataset-len", type=int, default=60000)
    ap.add_argument("--stepwise", action="store_true",
                    help="drive every phase of every step by RPC (the reference protocol)")
    ap.add_argument("--grad-comp-threshold", type=float, default=0.0)
    ap.add_argument("--out", type=str, default="")
    ap.add_argument("--checkpoint-dir", default="",
                    help="write a checkpoint per rank after every epoch (trainer/resume.py)")
    ap.add_argument("--resume", action="store_true",
                    help="continue from the newest epoch every rank has a checkpoint of")
    ap.add_argument("--fail-at-epoch", type=int, default=-1,
                    help="rank 1 raises once at the start of this epoch (recovery demo / test)")
    ap.add_argument("--model", default="lenet", choices=["lenet", "mixer"],
                    help="mixer: MLP-Mixer (the reference's train_nklc_nccl_mnist_3_mlpmx.py)")
    ap.add_argument("--loader", default="ngn", choices=["ngn", "queue", "shm", "obj"],
                    help="see dtloader.py (shm = the reference's train_ngn_mnist_2_dtpt.py)")
    ap.add_argument("--loader-workers", type=int, default=2)
    args = ap.parse_args()

    tmode = args.tmode or ("dp" if args.world_size > 1 else "no")
    pg_cfg = pg_cfg_from_args(args)
    ncclgrp.init_nccl_groups_map(tmode, pg_cfg)

    from necklace_b200.trainer import resume as nkresume
    if args.role == "scheduler":
        done = nkresume.resume_epoch(args.checkpoint_dir, args.world_size) if args.resume else 0
        cfg = {"role": "scheduler", "url": args.url, "workers": args.world_size,
               "start_epoch": done,
               "wdsz": args.world_size, "rank": 0, "epochs": args.epochs,
               "nccl_allreduce_typ": "grad", "stepwise": args.stepwise,
               "nccl_groups_grp_map": ncclgrp.get_nccl_groups_map_grp_dict()}
        svc = tndsnc.SVCScheduler(cfg)
        svc.loop()
        print("scheduler:", svc.exit_status)
        return 0 if svc.exit_status == "finished" else 1

    use_cuda = torch.cuda.is_available() and not args.no_cuda
    necklace_b200.init(args.gpu_rank)
    ctx = torch.device("cuda", int(args.gpu_rank)) if use_cuda else torch.device("cpu")
    torch.manual_seed(args.seed)
    if args.model == "mixer":
        from necklace_b200.models.mlp_mixer import MLPMixer
        net = MLPMixer(n_parts=2, seed=args.seed)
    else:
        net = LeNet()
    opt = torch.optim.SGD(net.parameters(), lr=args.lr, momentum=args.momentum)

    def dataloader_creator(rank, world):
        from dtloader import make_loader
        ds = SyntheticDataset(args.dataset_len, (1, 28, 28), classes=10, seed=args.seed)
        return make_loader(args.loader, ds, args.batch_size, rank, world, args.loader_workers)

    trainer_cfg = {
        "kn": args.world_size, "ti": args.rank, "ctx": ctx, "net": net, "opt": opt,
        "loss": WrpDoLoss(net, ctx), "batch_size": args.batch_size, "epochs": args.epochs,
        "dataset_len": args.dataset_len, "dataloader_type": "dp",
        "dataloader_creator": dataloader_creator,
        "dataloader_creator_args": (args.rank, args.world_size),
        "log_interval": args.log_interval, "tmode": tmode, "pg_cfg": pg_cfg,
        "comm_type": "gloo" if not use_cuda else args.comm_type,
        "grad_comp_cfg": ({"grad_comp_threshold": args.grad_comp_threshold,
                           "grad_size_threshold": 0} if args.grad_comp_threshold > 0 else None),
    }
    cfg = {"role": "worker", "url": args.url, "scheduler_url": args.server_url,
           "rank": args.rank, "trainer_cls": TrainerOPPytorch, "trainer_cfg": trainer_cfg}
    svc = tndsnc.SVCWorker(cfg)
    hook = HookLogLoss(net, ctx, args.out)
    svc.svr.trnr.register_hook_after_batch(hook.on_batch)
    svc.svr.trnr.register_hook_after_epoch(hook)
    if args.checkpoint_dir:
        done = nkresume.attach(svc.svr.trnr, args.checkpoint_dir, args.world_size, args.resume)
        if done:
            print(f"worker {args.rank}: resumed after {done} epoch(s)", flush=True)
    if args.fail_at_epoch >= 0 and args.rank == 1:
        marker = os.path.join(args.checkpoint_dir or ".", "failed_once")

        def fail_once(trnr, *a, **k):           # host-side fault injection
            if trnr.e == args.fail_at_epoch and not os.path.exists(marker):
                open(marker, "w").close()
                raise RuntimeError(f"injected failure at the start of epoch {trnr.e}")
        svc.svr.trnr.register_hook_before_epoch(fail_once)
    svc.loop()
    print(f"worker {args.rank}:", svc.exit_status)
    return 0 if svc.exit_status == "stopped" else 1


if __name__ == "__main__":
    sys.exit(main())
