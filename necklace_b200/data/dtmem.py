"""Shared-memory loader for batches of arbitrary picklable objects, under the reference's
module name (necklace/data/dtmem.py exports ``DataLoaderSharedMemory``): worker processes
pickle each collated batch into a ring of POSIX shared-memory slots (``data.shmem``)."""
from .loaders import ShmObjectRingDataLoader as DataLoaderSharedMemory  # noqa: F401
