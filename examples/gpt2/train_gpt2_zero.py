"""GPT-2 training with the whole-step engine in ``dp+zr`` mode (one process per GPU).

    python train_gpt2_zero.py --model tiny --steps 20                      # one GPU
    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        train_gpt2_zero.py --model medium --steps 50                         # eight GPUs

Every step (forward, backward, gradient reduce-scatter, sharded Adam on fp32 master
weights, parameter all-gather) runs inside the worker; the ZeRO part is one fused
peer-memory kernel.  Data is synthetic unless ``--tokens file.bin`` (uint16 token ids) is
given.  ``--ckpt path`` saves a consolidated, re-shardable checkpoint at the end and
resumes from it when it exists.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import numpy as np
import torch
import torch.distributed as dist

from necklace_b200 import checkpoint as ck
from necklace_b200.comm.symm import SymmetricHeap
from necklace_b200.models.gpt2 import GPT2, GPT2Config
from necklace_b200.parallel.engine import OptimConfig, TrainEngine


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny", choices=["tiny", "medium"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--tokens", default="")
    ap.add_argument("--ckpt", default="")
    ap.add_argument("--graph", action="store_true", help="capture the step in a CUDA graph")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = GPT2Config.medium() if args.model == "medium" else GPT2Config.tiny()
    torch.manual_seed(0)
    model = GPT2(cfg, device=dev)
    heap = group = None
    if world > 1:
        heap = SymmetricHeap(int(model.num_params() * 4.1) + (64 << 20))
        group = heap.peer_group()
    eng = TrainEngine(model, mode="zero" if world > 1 else "local", group=group, heap=heap,
                      optim=OptimConfig("adam", lr=args.lr, beta2=0.95, weight_decay=0.1),
                      use_cuda_graph=args.graph)
    if args.ckpt and os.path.exists(args.ckpt):
        meta = ck.load_engine_state(eng, ck.load(args.ckpt))
        if rank == 0:
            print("resumed from", args.ckpt, "at step", meta["step"])
    S = cfg.max_seq
    data = np.fromfile(args.tokens, dtype=np.uint16) if args.tokens else None
    g = torch.Generator().manual_seed(1000 + rank)
    for step in range(args.steps):
        if data is not None:
            off = torch.randint(0, len(data) - S - 1, (args.micro_batch,), generator=g)
            tok = torch.stack([torch.from_numpy(data[o:o + S + 1].astype(np.int64)) for o in off])
        else:
            tok = torch.randint(0, cfg.vocab, (args.micro_batch, S + 1), generator=g)
        tok = tok.pin_memory().to(dev, non_blocking=True)
        loss = eng.step(tok[:, :-1].contiguous(), tok[:, 1:].contiguous())
        if rank == 0 and (step % 10 == 0 or step == args.steps - 1):
            print(f"step {eng.step_count} loss {float(loss):.4f}", flush=True)
    eng.check()
    if args.ckpt:
        state = ck.engine_state(eng)
        ck.save(state, args.ckpt, rank=rank)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
