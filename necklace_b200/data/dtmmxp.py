"""Shared-memory loader with per-worker queues under the reference's module name
(necklace/data/dtmmxp.py; MXNet NDArrays there, the tensor ring of ``data.loaders`` here)."""
from .loaders import ShmRingDataLoader as DataLoaderSharedMemory  # noqa: F401
