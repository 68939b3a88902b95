"""Lists of pickled Python objects in POSIX shared memory.

``SharedMemList`` holds ``obj_cnt`` fixed-size slots; ``SharedMemArray`` adds a shared
``int32`` table with the pickled size of every slot, so objects of different sizes (up to
``obj_size`` bytes) can be stored and read back exactly.  Another process attaches with the
segment's ``name``.  The reference builds the same two classes on ``posix_ipc`` + ``mmap``
(necklace/data/shmem.py:15-187); here they sit on the standard library's
``multiprocessing.shared_memory`` (also POSIX ``shm_open`` underneath), so no extra
package is needed."""
from __future__ import annotations

import pickle
import struct
from multiprocessing import shared_memory


class SharedMemList:
    def __init__(self, name: str | None = None, obj_size: int = 1, obj_cnt: int = 1):
        self.obj_size, self.obj_cnt = int(obj_size), int(obj_cnt)
        size = max(1, self.obj_size * self.obj_cnt)
        self._owner = name is None
        self._shm = shared_memory.SharedMemory(create=True, size=size) if name is None \
            else shared_memory.SharedMemory(name=name)
        self.name = self._shm.name
        self._buf = self._shm.buf

    # helpers with the reference's names -------------------------------------------------
    @classmethod
    def copy(cls, arr):
        return cls(obj_size=arr.obj_size, obj_cnt=arr.obj_cnt)

    zeros_like = copy

    @staticmethod
    def pck_dumps(o) -> bytes:
        return pickle.dumps(o, protocol=4)

    @staticmethod
    def pck_loads(s):
        return pickle.loads(s)

    @classmethod
    def bin_size(cls, o) -> int:
        return len(cls.pck_dumps(o))

    def write_to_memory(self, data: bytes, sk: int = 0) -> None:
        self._buf[sk:sk + len(data)] = data

    def read_from_memory(self, z: int = 0, sk: int = 0) -> bytes:
        return bytes(self._buf[sk:sk + z] if z else self._buf[sk:])

    def __len__(self):
        return self.obj_cnt

    def __getitem__(self, idx):
        return self.pck_loads(self.read_from_memory(self.obj_size, self.obj_size * idx))

    def __setitem__(self, idx, item):
        s = self.pck_dumps(item)
        if len(s) > self.obj_size:
            raise ValueError(f"object needs {len(s)} bytes, slots hold {self.obj_size}")
        self.write_to_memory(s, self.obj_size * idx)

    def close(self):
        self._buf = None
        try:
            self._shm.close()
        except Exception:  # noqa: BLE001
            pass

    def unlink(self):
        try:
            self._shm.unlink()
        except FileNotFoundError:
            pass

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass


class SharedMemArray(SharedMemList):
    """``name`` (to attach) is ``"<data segment>:<size-table segment>"``."""

    def __init__(self, name: str | None = None, obj_size: int = 1, obj_cnt: int = 1):
        data_name = size_name = None
        if name is not None:
            data_name, size_name = name.split(":")
        super().__init__(data_name, obj_size, obj_cnt)
        self._sizes = shared_memory.SharedMemory(create=True, size=max(4, 4 * self.obj_cnt)) \
            if size_name is None else shared_memory.SharedMemory(name=size_name)
        if size_name is None:
            self._sizes.buf[:4 * self.obj_cnt] = bytes(4 * self.obj_cnt)
        self.name = f"{self._shm.name}:{self._sizes.name}"

    def size_of(self, idx: int) -> int:
        return struct.unpack_from("i", self._sizes.buf, 4 * idx)[0]

    def __getitem__(self, idx):
        n = self.size_of(idx)
        if n <= 0:
            return None
        return self.pck_loads(self.read_from_memory(n, self.obj_size * idx))

    def __setitem__(self, idx, item):
        s = self.pck_dumps(item)
        if len(s) > self.obj_size:
            raise ValueError(f"object needs {len(s)} bytes, slots hold {self.obj_size}")
        self.write_to_memory(s, self.obj_size * idx)
        struct.pack_into("i", self._sizes.buf, 4 * idx, len(s))

    def close(self):
        super().close()
        try:
            self._sizes.close()
        except Exception:  # noqa: BLE001
            pass

    def unlink(self):
        super().unlink()
        try:
            self._sizes.unlink()
        except FileNotFoundError:
            pass
