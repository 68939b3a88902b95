"""GPT-2 in trainer mode ``dp+zr`` through the framework's own process model: one scheduler
and one worker per GPU started from this script, control plane over ZeroMQ, the ZeRO trainer
``zroppt.TrainerMPOPPytorch`` with ``engine='native'`` (uniform shards, fused reduce-scatter +
Adam + all-gather kernel) and the peer-memory communicator (``--comm_type peer``).

    python train_gpt2_necklace.py -r scheduler -w 2 -u ipc:///tmp/nk-svr.ipc -e 1
    python train_gpt2_necklace.py -r worker -w 2 -k 0 -g 0 -u ipc:///tmp/nk-w0.ipc \
        -s ipc:///tmp/nk-svr.ipc -t dp+zr -dpsz 1 -zrsz 2 -x peer --model medium
    python train_gpt2_necklace.py -r worker -w 2 -k 1 -g 1 -u ipc:///tmp/nk-w1.ipc \
        -s ipc:///tmp/nk-svr.ipc -t dp+zr -dpsz 1 -zrsz 2 -x peer --model medium

``net_map`` has one unit per layer (embedding, blocks, head) like the reference's ZeRO
examples (examples/zero/mnist/pytorch/train_mnist_zr_5_dpzr_2.py); the scheduler sends one
``run_epoch`` per epoch and the workers run all steps without further RPC.  With
``--time-steps K --time-warmup W`` the worker times exactly K steps with CUDA events
(synchronised on both sides) and writes the result to ``--out``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from collections import OrderedDict

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch

import necklace_b200
from necklace_b200.comm import groups as ncclgrp
from necklace_b200.models.gpt2 import GPT2, GPT2Config
from necklace_b200.trainer import tndszd
from necklace_b200.trainer.zroppd import TrainerMPOPPytorch
from necklace_b200.utils.argutils import attach_nk_args_parser, pg_cfg_from_args
from necklace_b200.utils.hookbase import NklcHookBase


class SyntheticTokenLoader:
    """``steps`` batches of uniform token ids in pinned host memory (inputs, next-token
    targets)."""

    def __init__(self, steps, batch, seq, vocab, seed):
        g = torch.Generator().manual_seed(seed)
        pool = [torch.randint(0, vocab, (batch, seq + 1), generator=g) for _ in range(4)]
        pin = torch.cuda.is_available()
        self.x = [t[:, :-1].contiguous() for t in pool]
        self.y = [t[:, 1:].contiguous() for t in pool]
        if pin:
            self.x, self.y = [t.pin_memory() for t in self.x], [t.pin_memory() for t in self.y]
        self.steps, self.batch_size = steps, batch
        self.dataset = range(steps * batch)

    def __len__(self):
        return self.steps

    def __iter__(self):
        for i in range(self.steps):
            yield self.x[i % 4], self.y[i % 4]


class HookTimeSteps(NklcHookBase):
    """Before the data batch of step W+1 and of step W+K+1: synchronise and record a CUDA
    event, so that exactly K whole steps lie in between."""

    def __init__(self, net, ctx, warmup, steps, out, world, batch):
        super().__init__(net, ctx)
        self.w, self.k, self.out, self.world, self.batch = warmup, steps, out, world, batch
        self.n, self.e0, self.e1, self.loss = 0, None, None, None

    def __call__(self, trnr, *args, **kwargs):
        self.n += 1
        cuda = torch.device(self.ctx).type == "cuda"
        if self.n == self.w + 1:
            if cuda:
                torch.cuda.synchronize()
                self.e0 = torch.cuda.Event(enable_timing=True)
                self.e0.record()
            self.t0 = time.perf_counter()
        elif self.n == self.w + self.k + 1:
            if cuda:
                self.e1 = torch.cuda.Event(enable_timing=True)
                self.e1.record()
                torch.cuda.synchronize()
            self.loss = float(trnr.last_loss) if trnr.last_loss is not None else None
            ms = self.e0.elapsed_time(self.e1) if cuda else (time.perf_counter() - self.t0) * 1e3
            if self.out:
                with open(self.out + ".tmp", "w") as f:
                    json.dump({"rank": trnr.ti, "ms": ms, "steps": self.k, "loss": self.loss}, f)
                os.replace(self.out + ".tmp", self.out)


def main():
    ap = argparse.ArgumentParser()
    attach_nk_args_parser(ap)
    ap.add_argument("--model", default="tiny", choices=["tiny", "medium"])
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--steps-per-epoch", type=int, default=20)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--graph", action="store_true", help="capture the step in a CUDA graph")
    ap.add_argument("--bucket-mb", type=float, default=0.0)
    ap.add_argument("--time-steps", type=int, default=0)
    ap.add_argument("--time-warmup", type=int, default=3)
    ap.add_argument("--out", default="")
    ap.add_argument("--no-cuda", action="store_true", help="CPU run (gloo, fp32, tiny model)")
    args = ap.parse_args()

    world = args.world_size
    tmode = args.tmode or ("dp+zr" if world > 1 else "zr")
    pg_cfg = pg_cfg_from_args(args)
    if tmode == "dp+zr" and not pg_cfg.get("zr_size"):
        pg_cfg.update(dp_size=1, zr_size=world)
    ncclgrp.init_nccl_groups_map(tmode, pg_cfg)
    cfg_m = GPT2Config.medium() if args.model == "medium" else GPT2Config.tiny()
    steps = args.steps_per_epoch
    if args.time_steps:
        steps = args.time_warmup + args.time_steps + 1

    if args.role == "scheduler":
        n_units = cfg_m.n_layer + 2
        cfg = {"role": "scheduler", "url": args.url, "workers": world, "wdsz": world, "rank": 0,
               "epochs": args.epochs, "nccl_allreduce_typ": "dpzr" if world > 1 else "oozr",
               "net_map_maxlen": n_units,
               "nccl_groups_grp_map": ncclgrp.get_nccl_groups_map_grp_dict()}
        svc = tndszd.MPSVCScheduler(cfg)
        svc.loop()
        print("scheduler:", svc.exit_status, flush=True)
        return 0 if svc.exit_status == "finished" else 1

    gpu = int(args.gpu_rank)
    necklace_b200.init(gpu)
    use_cuda = torch.cuda.is_available() and not args.no_cuda
    if use_cuda:
        torch.cuda.set_device(gpu)
        ctx = torch.device("cuda", gpu)
    else:
        ctx = torch.device("cpu")
        cfg_m.dtype = torch.float32
    torch.manual_seed(0)
    model = GPT2(cfg_m, device=ctx)
    net_map = OrderedDict((i, {"net": u, "net_map_order": i, "worker_rank": i % world})
                          for i, u in enumerate(model.net_map_units()))
    S = cfg_m.max_seq
    nparam = model.num_params()
    trainer_cfg = {
        "kn": world, "ti": args.rank, "ctx": ctx, "net": None, "net_map": net_map,
        "net_map_order": args.rank, "net_map_maxlen": len(net_map), "loss": None,
        "engine": "native",
        "engine_kwargs": {"use_cuda_graph": args.graph,
                          "bucket_mb": args.bucket_mb if args.bucket_mb > 0 else None},
        "optimizer_params": {"kind": "adam", "lr": args.lr, "beta1": 0.9, "beta2": 0.95,
                             "eps": 1e-8, "weight_decay": 0.1},
        "batch_size": args.micro_batch, "epochs": args.epochs,
        "dataloader_creator": SyntheticTokenLoader,
        "dataloader_creator_args": (steps, args.micro_batch, S, cfg_m.vocab, 100 + args.rank),
        "log_interval": 10 ** 9 if args.time_steps else 10, "tmode": tmode, "pg_cfg": pg_cfg,
        "comm_type": "gloo" if not use_cuda else
        (args.comm_type if args.comm_type != "nccl" or world == 1 else "peer"),
        "heap_bytes": int(nparam * 2 * 2 * 1.02) + (64 << 20),
    }
    cfg = {"role": "worker", "url": args.url, "scheduler_url": args.server_url, "rank": args.rank,
           "trainer_cls": TrainerMPOPPytorch, "trainer_cfg": trainer_cfg}
    svc = tndszd.MPSVCWorker(cfg)
    if args.time_steps:
        hook = HookTimeSteps(None, ctx, args.time_warmup, args.time_steps, args.out, world,
                             args.micro_batch)
        svc.svr.trnr.register_hook_before_data_batch(hook)
    svc.loop()
    print(f"worker {args.rank}:", svc.exit_status, flush=True)
    return 0 if svc.exit_status == "stopped" else 1


if __name__ == "__main__":
    sys.exit(main())
