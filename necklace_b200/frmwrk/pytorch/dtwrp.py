"""DataLoader wrapper under the reference's module name (necklace/frmwrk/pytorch/dtwrp.py:7-30).
The reference patches the worker-index dispatch of an old torch iterator so that indices are
handed out lazily, one batch at a time; current torch dispatches that way already (bounded by
``prefetch_factor``), so the wrapper is the stock loader with that bound at its minimum."""
from __future__ import annotations

import torch.utils.data


class DataLoaderWrp(torch.utils.data.DataLoader):
    def __init__(self, *args, **kwargs):
        if kwargs.get("num_workers", 0) > 0:
            kwargs.setdefault("prefetch_factor", 2)
        super().__init__(*args, **kwargs)


def DataLoaderIterWrp(loader):
    """The iterator of a ``DataLoaderWrp`` (the reference exposes the iterator class)."""
    return iter(loader)
