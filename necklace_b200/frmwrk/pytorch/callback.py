"""Checkpoint and learning-rate callbacks (reference: necklace/frmwrk/pytorch/callback.py:16-26).
``adjust_learning_rate`` takes the base rate explicitly (the reference reads an
undefined global)."""
from __future__ import annotations

import shutil

import torch


def save_checkpoint(state, is_best, filename="checkpoint.pth.tar", best="model_best.pth.tar"):
    torch.save(state, filename)
    if is_best:
        shutil.copyfile(filename, best)


def adjust_learning_rate(optimizer, epoch, base_lr, decay=0.1, every=30):
    """lr = base_lr * decay ** (epoch // every)"""
    lr = base_lr * (decay ** (epoch // every))
    for g in optimizer.param_groups:
        g["lr"] = lr
    return lr
