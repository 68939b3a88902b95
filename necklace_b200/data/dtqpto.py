"""Queue-based multi-process loader under the reference's module name
(necklace/data/dtqpto.py exports DataLoaderSharedMemory)."""
from .loaders import QueueDataLoader as DataLoaderSharedMemory  # noqa: F401
