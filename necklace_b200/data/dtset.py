"""Dataset bases (reference: necklace/data/dtset.py:5-73) plus a synthetic dataset
used by the benchmarks (random tensors of a given shape, deterministic per index)."""
from __future__ import annotations

import random


class Dataset:
    def __getitem__(self, idx):
        raise NotImplementedError

    def __len__(self):
        raise NotImplementedError


class CacheDataset(Dataset):
    """Caches up to ``cache_num`` items of ``dt`` and evicts random ones when full."""

    def __init__(self, dt, num=None, cache_num=None, transform=None):
        self.dt, self.transform = dt, transform
        self.num = num if num is not None else len(dt)
        self.cache_num = cache_num if cache_num is not None else self.num
        self.cache = {}

    def __getitem__(self, idx):
        d = self.cache_get(idx)
        if d is None:
            d = self.one_item(idx)
            self.cache_put(idx, d)
        return d

    def __len__(self):
        return self.num

    def cache_get(self, idx):
        return self.cache.get(idx)

    def cache_put(self, idx, d):
        if len(self.cache) >= self.cache_num:
            self.cache_del_rand(max(1, self.cache_num // 10))
        self.cache[idx] = d

    def cache_del_rand(self, n):
        for k in random.sample(list(self.cache.keys()), min(n, len(self.cache))):
            del self.cache[k]

    def one_item(self, idx, *args, **kwargs):
        d = self.dt[idx]
        return self.transform(d) if self.transform else d


class SyntheticDataset(Dataset):
    """``(data, label)`` pairs drawn from a seeded generator keyed by the index.

    kind ``"image"``: fp32 tensor of ``shape`` (uniform [0,1) or N(0,1)), label uniform in
    ``[0, classes)``; kind ``"tokens"``: ``shape[0] + 1`` token ids split into input / target."""

    def __init__(self, length, shape, classes=10, kind="image", normal=False, seed=0):
        self.length, self.shape, self.classes = length, tuple(shape), classes
        self.kind, self.normal, self.seed = kind, normal, seed

    def __len__(self):
        return self.length

    def __getitem__(self, idx):
        import torch
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + int(idx))
        if self.kind == "tokens":
            t = torch.randint(0, self.classes, (self.shape[0] + 1,), generator=g)
            return t[:-1], t[1:]
        x = torch.randn(self.shape, generator=g) if self.normal else torch.rand(self.shape, generator=g)
        y = int(torch.randint(0, self.classes, (1,), generator=g))
        return x, y
