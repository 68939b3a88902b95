"""Central-sampler index arithmetic (reference: necklace/data/dtwrp.py:147-157):
with ``k`` ranks and batch size ``b``, batch ``i`` of rank ``r`` is the slice
``[i*b*k + r*b, i*b*k + (r+1)*b)`` of one global sampler."""
from __future__ import annotations

import types

import numpy as np

from .sampler import SliceSampler


# -- small data helpers (reference: necklace/data/dtwrp.py:19-64) -------------------------------
def is_generator(a):
    return isinstance(a, types.GeneratorType)


def is_iterator(a):
    return hasattr(a, "__iter__")


def get_len(a):
    if not hasattr(a, "__len__"):
        raise Exception("No __len__ defined")
    return len(a)


def np_is_ndarray(d):
    return isinstance(d, np.ndarray)


def np_array(d):
    return d if isinstance(d, np.ndarray) else np.array(d)


def label_to_onehot(y, shp):
    """``shp = (rows, classes)``: one row per label with a 1.0 at the label's column."""
    out = np.zeros(shp)
    out[np.arange(shp[0]), np.asarray(y, dtype=int)] = 1.0
    return out


# -- dataset wrappers (reference: necklace/data/dtwrp.py:93-121) -------------------------------
class DatasetBase:
    def __getitem__(self, idx):
        raise NotImplementedError

    def __len__(self):
        raise NotImplementedError


class DatasetWrp(DatasetBase):
    """Several parallel sequences (data, labels, ...) as one dataset: item ``i`` is the list of
    every sequence's element ``i``."""

    def __init__(self, ds, *args, **kwargs):
        self.ds = ds

    def __getitem__(self, idx):
        return [d[idx] for d in self.ds]

    def __len__(self):
        return len(self.ds[0])


class DataLoaderBase:
    """A loader that defines ``get_batch_by_dbi(dbi, dbf=None)`` is asked for its batches
    directly by ``DataLoaderWrp.get_data_batch``."""


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
        direct = getattr(self.loader, "get_batch_by_dbi", None)
        if direct is not None:
            return direct(dbi, dbf)
        items = [self.ds[i] for i in dbi]
        return dbf(items) if dbf else items
