"""Tensor stack / split / copy helpers (reference: necklace/frmwrk/pytorch/pttsutils.py:17-66)."""
from __future__ import annotations

import torch


def pt_ts_vstack(seq):
    return torch.cat(list(seq), dim=0)


def pt_ts_hstack(seq):
    return torch.cat(list(seq), dim=1)


def pt_ts_vsplit(a, n):
    return torch.chunk(a, n, dim=0)


def pt_ts_hsplit(a, n):
    return torch.chunk(a, n, dim=1)


def pt_ts_copy(x, requires_grad=None):
    y = x.detach().clone()
    y.requires_grad = x.requires_grad if requires_grad is None else requires_grad
    return y


def pt_is_tensor(x):
    return isinstance(x, torch.Tensor)
