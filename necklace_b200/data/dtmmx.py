"""Shared-memory loader under the reference's module name (necklace/data/dtmmx.py exports
``DataLoaderSharedMemory`` over MXNet NDArrays; here the tensor ring of ``data.loaders``)."""
from .loaders import ShmRingDataLoader as DataLoaderSharedMemory  # noqa: F401
