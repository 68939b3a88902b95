"""Drives the UNMODIFIED reference package (``baseline/_ref``) on the headline workload.

The reference's own ZeRO trainer (``necklace.trainer.zroppt.TrainerMPOPPytorch`` under the
``necklace.trainer.tndszr`` scheduler / worker services, exactly as in its example
``examples/zero/mnist/pytorch/train_mnist_zr_1.py``) trains GPT-2 medium on synthetic tokens:
one scheduler process, one worker process per GPU, ``net_map`` with one sub-module per
worker (the reference's ZeRO is layer-granular: sub-module i is owned by rank i).  The user
model is plain ``torch.nn`` (the modules of ``baseline/torch_gpt2.py``) with bf16 autocast
inside each part's forward, fp32 parameters (= master weights) and ``torch.optim.AdamW``
from the user's ``optimizer_creator``, which is how a user of the reference would get
"bf16 with fp32 master weights".  Nothing of necklace_b200 is imported here.

Run by ``bench.py --impl reference``; roles: ``scheduler`` or ``worker``.  A worker times
exactly ``--steps`` optimizer steps after ``--warmup`` with CUDA events (synchronised on both
sides) from the trainer's after-train-step hook and writes one JSON file.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from collections import OrderedDict

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "shims"))
sys.path.insert(0, os.path.join(HERE, "_ref"))
sys.path.insert(0, HERE)

import torch  # noqa: E402
import torch.nn as nn  # noqa: E402
import torch.nn.functional as F  # noqa: E402


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--role", required=True)
    ap.add_argument("--world", type=int, default=1)
    ap.add_argument("--rank", type=int, default=0)
    ap.add_argument("--gpu", type=int, default=0)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--model", default="gpt2-medium")
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--url", default="ipc:///tmp/nkref-wkr-0.ipc")
    ap.add_argument("--server-url", default="ipc:///tmp/nkref-svr.ipc")
    ap.add_argument("--out", default="")
    return ap.parse_args()


# ------------------------------------------------------------------ model parts (plain torch)
class PartFirst(nn.Module):
    def __init__(self, c, blocks):
        super().__init__()
        vp = (c["vocab"] + 127) // 128 * 128
        self.wte = nn.Embedding(vp, c["d_model"])
        nn.init.normal_(self.wte.weight, std=0.02)
        self.wpe = nn.Embedding(c["max_seq"], c["d_model"])
        self.blocks = nn.ModuleList(blocks)

    def embed(self, idx):
        S = idx.shape[1]
        return self.wte(idx) + self.wpe(torch.arange(S, device=idx.device))

    def forward(self, idx):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            x = self.embed(idx)
            for b in self.blocks:
                x = b(x)
        return x


class PartMid(nn.Module):
    def __init__(self, c, blocks):
        super().__init__()
        self.blocks = nn.ModuleList(blocks)

    def forward(self, x):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            for b in self.blocks:
                x = b(x)
        return x


class PartLast(nn.Module):
    """Blocks + final norm + output projection (its own weight: the reference's sub-modules
    live on different owners, so the projection cannot share the embedding matrix)."""

    def __init__(self, c, blocks):
        super().__init__()
        self.vocab = c["vocab"]
        self.blocks = nn.ModuleList(blocks)
        self.ln_f = nn.LayerNorm(c["d_model"])
        vp = (c["vocab"] + 127) // 128 * 128
        self.head = nn.Linear(c["d_model"], vp, bias=False)
        nn.init.normal_(self.head.weight, std=0.02)

    def forward(self, x):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            for b in self.blocks:
                x = b(x)
            return self.head(self.ln_f(x))[..., :self.vocab]


class PartWhole(PartFirst):
    """World size 1: the whole network is one sub-module and the projection is tied."""

    def __init__(self, c, blocks):
        super().__init__(c, blocks)
        self.vocab = c["vocab"]
        self.ln_f = nn.LayerNorm(c["d_model"])

    def forward(self, idx):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            x = self.embed(idx)
            for b in self.blocks:
                x = b(x)
            return F.linear(self.ln_f(x), self.wte.weight)[..., :self.vocab]


def build_net_map(model_name, world):
    from torch_gpt2 import CONFIGS, Block
    c = CONFIGS[model_name]
    torch.manual_seed(1234)
    blocks = [Block(c) for _ in range(c["n_layer"])]
    per = [len(blocks) // world + (1 if i < len(blocks) % world else 0) for i in range(world)]
    parts, k = [], 0
    for i in range(world):
        mine = blocks[k:k + per[i]]
        k += per[i]
        if world == 1:
            parts.append(PartWhole(c, mine))
        elif i == 0:
            parts.append(PartFirst(c, mine))
        elif i == world - 1:
            parts.append(PartLast(c, mine))
        else:
            parts.append(PartMid(c, mine))
    net_map = OrderedDict()
    for i, p in enumerate(parts):
        net_map[i] = {"net": p, "net_map_order": i, "worker_rank": i}
    return c, net_map


class SyntheticTokens(torch.utils.data.Dataset):
    def __init__(self, n, seq, vocab, seed):
        g = torch.Generator().manual_seed(seed)
        self.tok = torch.randint(0, vocab, (n, seq + 1), generator=g)

    def __len__(self):
        return self.tok.shape[0]

    def __getitem__(self, i):
        return self.tok[i, :-1], self.tok[i, 1:]


def main():
    args = parse()
    from necklace.rpc import ilog  # noqa: F401
    from necklace.trainer import tndszr
    c, net_map = build_net_map(args.model, args.world)
    S = min(args.seq, c["max_seq"])
    total_steps = args.warmup + args.steps

    if args.role == "scheduler":
        cfg = {"role": "scheduler", "url": args.server_url, "workers": args.world,
               "wdsz": args.world, "rank": 0, "epochs": 1, "nccl_allreduce_typ": "grad",
               "net_map": net_map}
        tndszr.MPSVCScheduler(cfg).loop()
        return 0

    import necklace
    from necklace.utils import hookbase, wrpbase
    try:
        necklace.init(args.gpu)          # numba device selection, as the examples do
    except Exception as e:  # noqa: BLE001
        print("necklace.init skipped:", e, flush=True)
    torch.cuda.set_device(args.gpu)
    from necklace.trainer import zroppt
    ctx = torch.device(args.gpu)
    vocab = c["vocab"]
    state = {"n": 0, "ev0": None, "ev1": None, "loss": None, "first": None}

    class Loss(wrpbase.NklcWrapperBase):
        def __call__(self, output, target, *a, **k):
            loss = F.cross_entropy(output.float().view(-1, vocab), target.view(-1))
            state["loss"] = loss.item()          # device -> host read of every step's loss
            if state["first"] is None:
                state["first"] = state["loss"]
            return loss

    def finish():
        ms = state["ev0"].elapsed_time(state["ev1"]) if state["ev1"] is not None else None
        out = {"rank": args.rank, "ms": ms, "steps_seen": state["n"],
               "loss_first": state["first"], "loss_last": state["loss"]}
        if args.out:
            with open(args.out + ".tmp", "w") as f:
                json.dump(out, f)
            os.replace(args.out + ".tmp", args.out)
        print("REF_RESULT " + json.dumps(out), flush=True)

    class AfterStep(hookbase.NklcHookBase):
        def __call__(self, trnr, *a, **k):
            state["n"] += 1
            if state["n"] == args.warmup:
                torch.cuda.synchronize()
                state["ev0"] = torch.cuda.Event(enable_timing=True)
                state["ev0"].record()
            elif state["n"] == total_steps:
                state["ev1"] = torch.cuda.Event(enable_timing=True)
                state["ev1"].record()
                torch.cuda.synchronize()
                # The measurement is complete.  Leave here instead of through the reference's
                # own shutdown: with one worker its scheduler never reaches the stop check
                # (the check sits in the branch taken while acks are still outstanding,
                # necklace/trainer/tndszr.py:1106-1117, :1806-1814) and would train forever.
                finish()
                sys.stdout.flush()
                os._exit(0)

    def make_opt(model, *a, **k):
        return torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), eps=1e-8,
                                 weight_decay=0.1)

    def make_loader(*a, **k):
        ds = SyntheticTokens((total_steps + 2) * args.micro_batch, S, vocab, 100 + args.rank)
        return torch.utils.data.DataLoader(ds, batch_size=args.micro_batch, shuffle=False,
                                           pin_memory=True, num_workers=0)

    net = net_map[args.rank]["net"]
    cfg = {
        "role": "worker", "url": args.url, "workers": args.world, "wdsz": args.world,
        "rank": args.rank, "scheduler_url": args.server_url,
        "trainer_cls": zroppt.TrainerMPOPPytorch,
        "trainer_cfg": {
            "kn": args.world, "ti": args.rank, "ctx": ctx, "net": net, "net_map": net_map,
            "net_init": None, "net_map_order": args.rank, "net_map_maxlen": len(net_map),
            "opt": make_opt(net), "optimizer_creator": make_opt, "optimizer_creator_args": (),
            "optimizer_creator_kwargs": {}, "loss": Loss(net, ctx), "mtrc": None,
            "optimizer_params": None, "epochs": 1, "batch_size": args.micro_batch,
            "dataloader_creator": make_loader, "dataloader_creator_args": (),
            "dataloader_creator_kwargs": {}, "use_dist_data_sampler": False,
            "log_interval": 1000000,
        },
    }
    svc = tndszr.MPSVCWorker(cfg)
    svc.svr.trnr.register_hook_after_do_a_train_step(AfterStep(net, ctx))
    svc.loop()
    finish()          # only reached if the epoch ended before the requested number of steps
    return 0


if __name__ == "__main__":
    rc = main()
    sys.stdout.flush()
    os._exit(rc)      # service threads of the RPC stand-ins are daemons; leave at once
