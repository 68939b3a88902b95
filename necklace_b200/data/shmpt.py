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


# dtype names of the reference's tables (necklace/data/shmpt.py:150-205)
_BY_NAME = {"torch.float": torch.float32, "torch.float32": torch.float32,
            "torch.double": torch.float64, "torch.float64": torch.float64,
            "torch.half": torch.float16, "torch.float16": torch.float16,
            "torch.uint8": torch.uint8, "torch.int8": torch.int8, "torch.short": torch.int16,
            "torch.int16": torch.int16, "torch.int": torch.int32, "torch.int32": torch.int32,
            "torch.long": torch.int64, "torch.int64": torch.int64}
_TENSOR_TYPES = {torch.float32: "FloatTensor", torch.float64: "DoubleTensor",
                 torch.float16: "HalfTensor", torch.uint8: "ByteTensor", torch.int8: "CharTensor",
                 torch.int16: "ShortTensor", torch.int32: "IntTensor", torch.int64: "LongTensor"}


def _dtype(d):
    return _BY_NAME[d] if isinstance(d, str) else d


def dtype_to_tensor(dtype, use_cuda=False):
    """The legacy tensor class of a dtype name (``'torch.float'`` -> ``torch.FloatTensor``)."""
    mod = torch.cuda if use_cuda else torch
    return getattr(mod, _TENSOR_TYPES[_dtype(dtype)])


def dtype_to_storage(dtype, use_cuda=False):
    """The storage behind tensors is untyped in current torch; the reference's typed storage
    classes have no counterpart, so this returns ``torch.UntypedStorage``."""
    return torch.UntypedStorage


class SharedMemArray:
    """``SharedMemArray(shape, dtype)`` creates, ``SharedMemArray.attach(*key)`` attaches.  The
    reference's call shape works too: ``SharedMemArray(name=None, obj_shape=..., dtype='torch.
    float', sk=None)`` creates when ``sk`` is ``None`` and attaches to the key ``sk`` otherwise;
    ``.sk`` is the key, ``.buf`` the tensor, ``unlink()`` releases (necklace/data/shmpt.py:209-295)."""

    def __init__(self, shape=None, dtype=torch.float32, name=None, create=True, *, obj_shape=None,
                 obj_cnt=1, gpu_i=0, sk=None, use_cuda=False):
        if shape is None or isinstance(shape, str):       # the reference's (name, obj_shape, ...)
            shape = obj_shape if obj_shape is not None else (1,)
        if sk is not None:
            name, create = sk[0], False
            shape = sk[1] if obj_shape is None else obj_shape
        dtype = _dtype(dtype)
        self.shape, self.dtype = tuple(shape), dtype
        self.obj_shape, self.obj_cnt = self.shape, obj_cnt
        npdt = np.dtype(_NP[dtype])
        nbytes = max(1, int(np.prod(self.shape)) * npdt.itemsize)
        self.shm = shared_memory.SharedMemory(name=name, create=create, size=nbytes)
        self._owner = create
        arr = np.ndarray(self.shape, dtype=npdt, buffer=self.shm.buf)
        self.tensor = torch.from_numpy(arr)
        if create:
            self.tensor.zero_()

    @property
    def key(self):
        """What another process needs to attach: ``SharedMemArray.attach(*key)``."""
        return (self.shm.name, self.shape, self.dtype)

    sk = key

    @property
    def buf(self):
        return self.tensor

    @classmethod
    def attach(cls, name, shape, dtype):
        return cls(shape, dtype, name=name, create=False)

    @classmethod
    def create_from_shmem_key(cls, sk=None, shape=None, dtype=None):
        if not sk:
            raise Exception("no shmem key given")
        return cls(sk[1] if shape is None else shape, sk[2] if dtype is None else dtype,
                   name=sk[0], create=False)

    @classmethod
    def ndarray_from_shmem_key(cls, sk, shape=None, dtype=None):
        a = cls.create_from_shmem_key(sk, shape, dtype)
        _KEEP.append(a)
        return a.tensor

    @classmethod
    def create_mx_ndarray_shmem(cls, shape, dtype="torch.float"):
        a = cls(shape, dtype)
        _KEEP.append(a)
        return a.key, a.tensor

    def __getitem__(self, idx):
        return self.tensor[idx]

    def __setitem__(self, idx, item):
        self.tensor[idx] = torch.as_tensor(item)

    def close(self):
        self.tensor = None
        try:
            self.shm.close()
            if self._owner:
                self.shm.unlink()
        except Exception:  # noqa: BLE001
            pass

    unlink = close


_KEEP: list = []


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
