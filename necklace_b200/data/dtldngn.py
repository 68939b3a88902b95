"""Single-process loader with a re-shardable batch sampler
(reference: necklace/data/dtldngn.py:8-69).  ``_attr_ngn_dataloader`` marks loaders
whose sampler the trainer may replace with a rank's slice of a global shuffle."""
from __future__ import annotations

from .batchify import stack_batchify_fn
from .sampler import BatchSampler, SliceBatchSampler, SliceSampler


class DataLoaderNgnBase:
    _attr_ngn_dataloader = True

    def __init__(self, dataset, batch_size=None, shuffle=False, sampler=None, last_batch=None,
                 batch_sampler=None, batchify_fn=None, seed=None):
        self.dataset, self.batch_size, self.shuffle = dataset, batch_size, shuffle
        self.last_batch = last_batch or "keep"
        self.batchify_fn = batchify_fn or stack_batchify_fn
        if batch_sampler is None:
            if sampler is None:
                sampler = SliceSampler(len(dataset), shuffle=shuffle, seed=seed)
            batch_sampler = self._make_batch_sampler(sampler)
        self.batch_sampler = batch_sampler

    def init_slice_sampler(self):
        """(Re)create the default sampler over the whole dataset and its batch sampler
        (reference: necklace/data/dtldngn.py:37-39)."""
        self.sampler = SliceSampler(len(self.dataset), shuffle=self.shuffle)
        self.batch_sampler = self._make_batch_sampler(self.sampler)

    def _make_batch_sampler(self, smplr):
        cls = SliceBatchSampler if isinstance(smplr, SliceSampler) else BatchSampler
        return cls(smplr, self.batch_size, self.last_batch)

    def reset_batch_sampler(self, new_sampler, *args, **kwargs):
        self.batch_sampler = self._make_batch_sampler(new_sampler)

    def __len__(self):
        return len(self.batch_sampler)

    def __iter__(self):
        if self.shuffle:
            self.batch_sampler.shuffle()
        for batch in self.batch_sampler:
            yield self._get_a_batch(batch)

    def _get_a_batch(self, batch):
        return self.batchify_fn([self.dataset[i] for i in batch])

    def clear(self):
        pass
