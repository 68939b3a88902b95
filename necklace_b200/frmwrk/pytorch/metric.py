"""``AverageMeter`` and top-k ``accuracy`` (reference: necklace/frmwrk/pytorch/metric.py:10-42)."""
from __future__ import annotations

import torch


class AverageMeter:
    def __init__(self):
        self.reset()

    def reset(self):
        self.val = self.avg = self.sum = 0.0
        self.count = 0

    def update(self, val, n=1):
        self.val = val
        self.sum += val * n
        self.count += n
        self.avg = self.sum / max(self.count, 1)


def accuracy(output, target, topk=(1,)):
    with torch.no_grad():
        maxk = max(topk)
        _, pred = output.topk(maxk, 1, True, True)
        correct = pred.t().eq(target.view(1, -1).expand_as(pred.t()))
        return [correct[:k].reshape(-1).float().sum(0) * (100.0 / target.size(0)) for k in topk]


class Accuracy:
    """Metric object with the ``reset / update(target, output) / get`` protocol the
    trainers call (the reference follows MXNet's metric protocol,
    necklace/trainer/tnoppt.py:485-488, :566-568)."""

    def __init__(self, name="accuracy"):
        self.name = name
        self.reset()

    def reset(self):
        self.correct = self.total = 0

    def update(self, target, output):
        with torch.no_grad():
            self.correct += int((output.argmax(-1) == target).sum())
            self.total += int(target.numel())

    def get(self):
        return self.name, self.correct / max(self.total, 1)
