"""Megatron-style samplers (reference: necklace/frmwrk/pytorch/mpnn/samplers.py:24-140):
an epoch-seeded ``RandomSampler`` and a ``DistributedBatchSampler`` in which every
rank takes ``batch[rank*b/ws : (rank+1)*b/ws]`` of each global batch."""
from __future__ import annotations

import torch
from torch.utils import data


class RandomSampler(data.sampler.Sampler):
    def __init__(self, data_source, replacement=False, num_samples=None, seed=0):
        self.data_source, self.replacement = data_source, replacement
        self._num_samples, self.seed, self.epoch = num_samples, seed, -1

    @property
    def num_samples(self):
        return len(self.data_source) if self._num_samples is None else self._num_samples

    def __iter__(self):
        n = len(self.data_source)
        g = torch.Generator()
        if self.epoch >= 0:
            g.manual_seed(self.seed + self.epoch)
        if self.replacement:
            return iter(torch.randint(high=n, size=(self.num_samples,), generator=g).tolist())
        return iter(torch.randperm(n, generator=g).tolist())

    def __len__(self):
        return self.num_samples

    def set_epoch(self, epoch):
        self.epoch = epoch


class DistributedBatchSampler(data.sampler.BatchSampler):
    def __init__(self, sampler, batch_size, drop_last, rank=-1, world_size=2, wrap_last=False):
        super().__init__(sampler, batch_size, drop_last)
        if rank == -1:
            import torch.distributed as dist
            rank = dist.get_rank() if dist.is_initialized() else 0
        self.rank, self.world_size, self.wrap_last = rank, world_size, wrap_last
        self.sampler.wrap_around = 0
        self.start_iter = 0

    def __iter__(self):
        batch, i = [], 0
        for idx in self.data_iterator(self.sampler, wrap_around=False):
            batch.append(idx)
            if len(batch) == self.batch_size:
                if i >= self.start_iter:
                    yield self._batch(batch)
                i += 1
                batch = []
        if batch and not self.drop_last:
            if self.wrap_last:
                batch = (batch + batch * self.batch_size)[:self.batch_size]
            yield self._batch(batch)
        self.start_iter = 0

    def data_iterator(self, _iter, wrap_around=False):
        for idx in _iter:
            yield idx

    def _batch(self, batch):
        per = self.batch_size // self.world_size
        return batch[self.rank * per:(self.rank + 1) * per]
