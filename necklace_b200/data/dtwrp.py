"""Central-sampler index arithmetic (reference: necklace/data/dtwrp.py:147-157):
with ``k`` ranks and batch size ``b``, batch ``i`` of rank ``r`` is the slice
``[i*b*k + r*b, i*b*k + (r+1)*b)`` of one global sampler."""
from __future__ import annotations

from .sampler import SliceSampler


class SamplerWrp(SliceSampler):
    def __init__(self, length, shuffle=False, seed=None):
        super().__init__(length, shuffle=shuffle, seed=seed)


class DataLoaderWrp:
    def __init__(self, loader, ds, rank, mdtype=None, role="worker", batch_size=1, kn=1,
                 shuffle=False, seed=None):
        self.loader, self.ds, self.rank, self.role = loader, ds, rank, role
        self.b, self.k = batch_size, kn
        self.sampler = SamplerWrp(len(ds), shuffle=shuffle, seed=seed)

    def get_data_batch_index(self, rank, i, b=None, k=None):
        b, k = b or self.b, k or self.k
        lo = i * b * k + rank * b
        return self.sampler.indices[lo:lo + b]

    def get_data_batch(self, dbi, dbf=None):
        items = [self.ds[i] for i in dbi]
        return dbf(items) if dbf else items
