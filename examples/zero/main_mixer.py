"""Stock single-process counterpart of ``train_mnist_mixer_zr.py``: the same MLP-Mixer, data
and optimizer in a plain PyTorch loop (reference: examples/zero/mnist/pytorch/main_mlpmx.py).
Prints the mean loss of every epoch; ``--out`` writes them as JSON for comparison."""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch
import torch.nn as nn

from necklace_b200.data.dtset import SyntheticDataset
from necklace_b200.models.mlp_mixer import MLPMixer


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--epochs", "-e", type=int, default=1)
    ap.add_argument("--batch-size", "-b", type=int, default=32)
    ap.add_argument("--lr", type=float, default=0.05)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--dataset-len", type=int, default=256)
    ap.add_argument("--parts", type=int, default=3)
    ap.add_argument("--replicas", type=int, default=1,
                    help="emulate this many data-parallel replicas (gradient = sum over them)")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    net = MLPMixer(n_parts=args.parts, seed=args.seed)
    opt = torch.optim.SGD(net.parameters(), lr=args.lr)
    ds = SyntheticDataset(args.dataset_len, (1, 28, 28), classes=10, seed=args.seed)
    ce = nn.CrossEntropyLoss()
    per = args.dataset_len // args.replicas
    epoch_loss = []
    for _ in range(args.epochs):
        losses = []
        for i in range(per // args.batch_size):
            opt.zero_grad()
            tot = 0.0
            for r in range(args.replicas):
                idx = range(r * per + i * args.batch_size, r * per + (i + 1) * args.batch_size)
                x = torch.stack([ds[j][0] for j in idx])
                y = torch.tensor([ds[j][1] for j in idx])
                loss = ce(net(x), y) / args.replicas
                loss.backward()
                tot += float(loss)
            opt.step()
            losses.append(tot)
        epoch_loss.append(sum(losses) / len(losses))
        print("epoch loss", epoch_loss[-1])
    if args.out:
        json.dump({"epoch_loss": epoch_loss,
                   "weights_sum": float(sum(p.double().sum() for p in net.parameters()))},
                  open(args.out, "w"))
    return 0


if __name__ == "__main__":
    sys.exit(main())
