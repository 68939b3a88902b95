"""Dummy dataset / loader for ranks that receive their batch by broadcast
(non-zero members of a tensor-parallel group; reference: necklace/data/dtdummy.py:4-32).
It yields ``(None, None)`` once per batch so step counts stay aligned."""
from __future__ import annotations


class DtstDummy:
    def __init__(self, ds_len):
        self.ds_len = ds_len

    def __getitem__(self, idx=None):
        return None, None

    def __len__(self):
        return self.ds_len


class DtldDummy:
    def __init__(self, ds, batch_size, drop_last=True):
        self.dataset, self.batch_size, self.drop_last = ds, batch_size, drop_last
        n = len(ds)
        self.n = n // batch_size if drop_last else (n + batch_size - 1) // batch_size

    def __iter__(self):
        for _ in range(self.n):
            yield None, None

    def __len__(self):
        return self.n
