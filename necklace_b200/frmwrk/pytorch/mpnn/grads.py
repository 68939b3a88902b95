"""Gradient clipping by the global norm when parameters are split over the model-parallel
group (``clip_grad_norm`` is listed, commented out, among the exports of the reference's
``mpnn`` package, necklace/frmwrk/pytorch/mpnn/__init__.py:5).  Sharded parameters (tagged
``model_parallel`` by the parallel layers) contribute on every rank, replicated ones on the
group's rank 0 only, so nothing is counted twice."""
from __future__ import annotations

import torch

from ....comm import fns
from . import initialize as mpu


def clip_grad_norm(parameters, max_norm, norm_type=2):
    params = [p for p in ([parameters] if isinstance(parameters, torch.Tensor) else parameters)
              if p.grad is not None]
    ws, rank = mpu.get_model_parallel_world_size(), mpu.get_model_parallel_rank()
    group = mpu.get_model_parallel_group()
    counted = [p for p in params if getattr(p, "model_parallel", False) or rank == 0 or ws == 1]
    dev = params[0].grad.device if params else torch.device("cpu")
    norm_type = float(norm_type)
    if norm_type == float("inf"):
        total = torch.stack([p.grad.detach().abs().max().float() for p in counted]).max() \
            if counted else torch.zeros((), device=dev)
        if ws > 1:
            total = total.reshape(1)
            fns.all_reduce(total, op="max", group=group)
            total = total[0]
    else:
        total = sum((p.grad.detach().float().norm(norm_type) ** norm_type for p in counted),
                    torch.zeros((), device=dev))
        if ws > 1:
            total = total.reshape(1)
            fns.all_reduce(total, group=group)
            total = total[0]
        total = total ** (1.0 / norm_type)
    coef = float(max_norm) / (float(total) + 1e-6)
    if coef < 1:
        for p in params:
            p.grad.mul_(coef)
    return float(total)
