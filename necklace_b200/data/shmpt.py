"""Torch CPU tensors in named shared memory (attach from any process by name).

The reference shares tensors by torch's private storage filename handles
(necklace/data/shmpt.py:209-295); this uses ``multiprocessing.shared_memory``,
whose names are plain strings that travel in RPC messages."""
from __future__ import annotations

from multiprocessing import shared_memory

import numpy as np
import torch

_NP = {torch.float32: np.float32, torch.float64: np.float64, torch.float16: np.float16,
       torch.int64: np.int64, torch.int32: np.int32, torch.int16: np.int16, torch.int8: np.int8,
       torch.uint8: np.uint8, torch.bool: np.bool_}


class SharedMemArray:
    def __init__(self, shape, dtype=torch.float32, name=None, create=True):
        self.shape, self.dtype = tuple(shape), dtype
        npdt = np.dtype(_NP[dtype])
        nbytes = max(1, int(np.prod(self.shape)) * npdt.itemsize)
        self.shm = shared_memory.SharedMemory(name=name, create=create, size=nbytes)
        self._owner = create
        arr = np.ndarray(self.shape, dtype=npdt, buffer=self.shm.buf)
        self.tensor = torch.from_numpy(arr)

    @property
    def key(self):
        """What another process needs to attach: ``SharedMemArray.attach(*key)``."""
        return (self.shm.name, self.shape, self.dtype)

    @classmethod
    def attach(cls, name, shape, dtype):
        return cls(shape, dtype, name=name, create=False)

    def close(self):
        self.tensor = None
        try:
            self.shm.close()
            if self._owner:
                self.shm.unlink()
        except Exception:  # noqa: BLE001
            pass


class SharedMemList:
    """A fixed number of equally shaped shared tensors (ring slots)."""

    def __init__(self, n, shape, dtype=torch.float32):
        self.items = [SharedMemArray(shape, dtype) for _ in range(n)]

    def keys(self):
        return [a.key for a in self.items]

    def __getitem__(self, i):
        return self.items[i].tensor

    def __len__(self):
        return len(self.items)

    def close(self):
        for a in self.items:
            a.close()
