"""The loaders a data-parallel worker can feed from (counterpart of the reference's
examples/dp/mnist/pytorch/dtloader.py, which builds its shared-memory loader for
train_ngn_mnist_2_dtpt.py):

    ngn    in-process loader (`data.dtldngn.DataLoaderNgnBase`)
    queue  worker processes hand collated batches over queues (`data.dtqptp`)
    shm    worker processes write batches into rings of shared tensors (`data.dtmptv`)
    obj    worker processes pickle whole batches into POSIX shared memory (`data.dtmem`)

All take the same sampler, so a rank sees the same samples in the same order whichever
loader it uses."""
from necklace_b200.data.dtldngn import DataLoaderNgnBase
from necklace_b200.data.sampler import SliceSampler


def make_loader(kind, dataset, batch_size, rank, world, workers=2):
    per = len(dataset) // world
    sampler = SliceSampler(indices=list(range(rank * per, (rank + 1) * per)))
    if kind == "ngn":
        return DataLoaderNgnBase(dataset, batch_size=batch_size, sampler=sampler,
                                 last_batch="discard")
    if kind == "queue":
        from necklace_b200.data.dtqptp import DataLoaderSharedMemory as Loader
    elif kind == "shm":
        from necklace_b200.data.dtmptv import DataLoaderSharedMemory as Loader
    elif kind == "obj":
        from necklace_b200.data.dtmem import DataLoaderSharedMemory as Loader
    else:
        raise ValueError(f"unknown loader {kind!r}")
    kw = {}
    if kind == "obj":
        # the object ring carries whatever the collate function returns; here the stacked
        # (images, labels) pair, pickled as numpy-backed tensors (~63 KB per 20 images)
        from necklace_b200.data.batchify import stack_batchify_fn
        kw = {"inter_batchify_fn": stack_batchify_fn,
              "slot_bytes": 4 * (batch_size * 28 * 28 * 4 + 4096)}
    return Loader(dataset, batch_size, sampler=sampler, last_batch="discard",
                  num_workers=workers, part_num=4, **kw)
