"""Shared-memory ring loader under the reference's module name
(necklace/data/dtmptp.py exports DataLoaderSharedMemory; the pickled-object,
numpy and MXNet shared-memory variants of the reference collapse into the one
torch-tensor ring implementation)."""
from .loaders import ShmRingDataLoader as DataLoaderSharedMemory  # noqa: F401
