"""Shared-memory array under the reference's module name (necklace/data/shmmx.py:9-75).  The
reference shares an MXNet NDArray between processes and hands its shared-memory key around;
MXNet is not part of this build, so the array is a numpy array over a POSIX shared-memory
segment and the key ``sk`` is ``(segment name, shape, dtype string)``: picklable, attachable
from any process, same ``buf[idx]`` access."""
from __future__ import annotations

from multiprocessing import shared_memory

import numpy as np


class SharedMemArray(object):
    def __init__(self, name=None, obj_shape=(1,), obj_cnt=1, dtype=np.float32, sk=None):
        self.name, self.obj_shape, self.obj_cnt, self.dtype, self.sk = \
            name, tuple(obj_shape), obj_cnt, dtype, sk
        self._shm, self._owner = None, sk is None
        self.init_shms()
        self.init_bufs(self.sk)

    def init_shms(self):
        pass

    def init_bufs(self, sk=None):
        if sk is None:
            self.sk, self.buf, self._shm = self._create(self.obj_shape, self.dtype)
        else:
            self.buf, self._shm = self._attach(sk)
            self.obj_shape, self.dtype = tuple(sk[1]), np.dtype(sk[2])

    @staticmethod
    def _create(shape, dtype=np.float32):
        dt = np.dtype(dtype)
        nbytes = max(1, int(np.prod(shape)) * dt.itemsize)
        shm = shared_memory.SharedMemory(create=True, size=nbytes)
        arr = np.ndarray(shape, dtype=dt, buffer=shm.buf)
        arr[...] = 0
        return (shm.name, tuple(shape), dt.str), arr, shm

    @staticmethod
    def _attach(sk):
        shm = shared_memory.SharedMemory(name=sk[0])
        return np.ndarray(tuple(sk[1]), dtype=np.dtype(sk[2]), buffer=shm.buf), shm

    @classmethod
    def ndarray_from_shmem_key(cls, sk):
        """The array behind a key (the segment stays mapped as long as the array lives)."""
        arr, shm = cls._attach(sk)
        _KEEP.append(shm)
        return arr

    @classmethod
    def create_from_shmem_key(cls, sk=None):
        if not sk:
            raise Exception("no shmem key given")
        return cls(sk=sk)

    def unlink(self):
        """Called by the creator to release the segment."""
        self.buf = None
        if self._shm is not None:
            self._shm.close()
            if self._owner:
                try:
                    self._shm.unlink()
                except FileNotFoundError:
                    pass
            self._shm = None

    def __getitem__(self, idx):
        return self.buf[idx]

    def __setitem__(self, idx, item):
        self.buf[idx] = item


_KEEP: list = []
