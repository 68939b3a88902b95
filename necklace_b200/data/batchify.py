"""Collate helpers (reference: necklace/data/batchify.py:16-50)."""
from __future__ import annotations

import numpy as np


def identity_batchify_fn(dt):
    return dt


def label_mod_batchify_fn(n):
    def fn(dt):
        data, label = dt
        return data, label % n
    return fn


def np2pt_batchify_fn(dt):
    import torch
    data, label = dt
    return torch.from_numpy(np.asarray(data)), torch.from_numpy(np.asarray(label)).long()


def pt_batchify_fn(dt):
    from torch.utils.data import default_collate
    return default_collate(dt)


def flt2int_bchfn(dt):
    data, label = dt
    return data, label.long()


def stack_batchify_fn(items):
    """List of ``(data, label)`` samples -> ``(data[B,...], label[B])`` tensors."""
    import torch
    xs, ys = zip(*items)
    xs = torch.stack([x if isinstance(x, torch.Tensor) else torch.as_tensor(x) for x in xs])
    ys = torch.stack([y if isinstance(y, torch.Tensor) else torch.as_tensor(y) for y in ys])
    return xs, ys


def nothing_batchify_fn(dt):
    """The batch as it is (reference: necklace/data/batchify.py:16-17)."""
    return dt


def label_reduce_batchify_fn(dt, lbl_n=1000):
    """Fold the first label column into ``[0, lbl_n)`` in place (reference:
    necklace/data/batchify.py:20-23): ``dt = (data, labels[B, k])``."""
    for row in dt[1]:
        row[0] %= lbl_n
    return dt
