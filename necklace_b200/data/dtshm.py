"""Shared-memory loader for batches of arbitrary picklable objects, under the reference's
module name (necklace/data/dtshm.py exports ``DataLoaderSharedMemory``): worker processes
pickle each collated batch into a ring of POSIX shared-memory slots (``data.shmem``)."""
from .loaders import ShmObjectRingDataLoader as DataLoaderSharedMemory  # noqa: F401


class DataLoaderShmForModule(DataLoaderSharedMemory):
    """With the ``provide_data`` / ``provide_label`` descriptors an MXNet ``Module`` asks its
    iterator for: ``[(name, shape)]`` of one training batch, from the first sample."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.mode = "train"
        first = self.dataset[0]
        self.data, self.label = first[0], first[1]

    @property
    def provide_data(self):
        return [("data", (self.batch_size,) + tuple(getattr(self.data, "shape", ())))]

    @property
    def provide_label(self):
        return [("label", (self.batch_size,))]

    def reset(self):
        pass
