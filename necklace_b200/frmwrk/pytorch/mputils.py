"""``ModelPartWrapper``: one pipeline stage (reference: necklace/frmwrk/pytorch/mputils.py:11-66).

Stages after the first detach their inputs and mark them ``requires_grad`` so that the
gradient with respect to the stage input can be read after backward and sent to the
previous stage; the stage output is cached for ``mp_backward(grads)``."""
from __future__ import annotations

import torch
import torch.nn as nn


def _as_list(x):
    if x is None:
        return []
    return list(x) if isinstance(x, (list, tuple)) else [x]


class ModelPartWrapper(nn.Module):
    def __init__(self, submodules, mp_order=0, *args, **kwargs):
        super().__init__()
        mods = _as_list(submodules)
        self.net = mods[0] if len(mods) == 1 else nn.Sequential(*mods)
        self.mp_order = mp_order
        self.inputs = None
        self.output = None

    def cache_graded_input(self, *inputs):
        if self.mp_order == 0:
            self.inputs = list(inputs)
            return self.inputs
        cached = []
        for x in inputs:
            if isinstance(x, torch.Tensor) and x.is_floating_point():
                x = x.detach()
                x.requires_grad_(True)
            cached.append(x)
        self.inputs = cached
        return cached

    def forward(self, *inputs):
        xs = self.cache_graded_input(*inputs)
        self.output = self.net(*xs)
        return self.output

    def get_input_grads(self):
        return [x.grad for x in (self.inputs or [])
                if isinstance(x, torch.Tensor) and x.requires_grad and x.grad is not None]

    def mp_backward(self, grads):
        outs = [o for o in _as_list(self.output) if isinstance(o, torch.Tensor)]
        gs = _as_list(grads)
        pairs = [(o, g) for o, g in zip(outs, gs) if o.requires_grad]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        self.output = None


class MpTrnrModulesMap:
    """``net_map`` helper: ordered stages with their owner ranks."""

    def __init__(self, net_map):
        self.net_map = net_map

    def orders(self):
        return sorted(self.net_map.keys())

    def worker_rank(self, order):
        return self.net_map[order].get("worker_rank")

    def net(self, order):
        return self.net_map[order].get("net")
