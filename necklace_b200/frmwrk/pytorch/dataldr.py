"""``get_dist_dataloader`` (reference: necklace/frmwrk/pytorch/dataldr.py:14-41):
a ``DistributedSampler`` shard of ``dataset`` for ``rank`` of ``world_size``."""
from __future__ import annotations

from torch.utils.data import DataLoader
from torch.utils.data.distributed import DistributedSampler


def get_dist_dataloader(dataset, world_size=1, rank=0, shuffle=True, num_workers=0,
                        pin_memory=False, batch_size=1, drop_last=False, seed=0, **kwargs):
    sampler = DistributedSampler(dataset, num_replicas=world_size, rank=rank, shuffle=shuffle,
                                 seed=seed, drop_last=drop_last)
    return DataLoader(dataset, batch_size=batch_size, shuffle=False, sampler=sampler,
                      num_workers=num_workers, pin_memory=pin_memory, drop_last=drop_last,
                      **kwargs)
