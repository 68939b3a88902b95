"""Index samplers (sequential, random, batch with last-batch policy, sliceable).

Same classes and semantics as the reference's Gluon-style samplers
(necklace/data/sampler.py:7-163): ``BatchSampler(last_batch=...)`` keeps, discards
or rolls the incomplete last batch over to the next epoch; ``SliceSampler`` holds an
explicit index list that can be sliced (``s[a:b]``) to shard it over ranks or loader
workers and reshuffled in place."""
from __future__ import annotations

import random


class Sampler:
    def __iter__(self):
        raise NotImplementedError

    def __len__(self):
        raise NotImplementedError

    def shuffle(self):
        pass


class SequentialSampler(Sampler):
    def __init__(self, length):
        self._length = length

    def __iter__(self):
        return iter(range(self._length))

    def __len__(self):
        return self._length


class RandomSampler(Sampler):
    def __init__(self, length, seed=None):
        self._length = length
        self._rng = random.Random(seed)

    def __iter__(self):
        idx = list(range(self._length))
        self._rng.shuffle(idx)
        return iter(idx)

    def __len__(self):
        return self._length


class BatchSampler(Sampler):
    def __init__(self, sampler, batch_size, last_batch="keep"):
        if last_batch not in ("keep", "discard", "rollover"):
            raise ValueError("last_batch must be one of 'keep', 'discard', 'rollover', "
                             f"got {last_batch!r}")
        self._sampler, self._batch_size, self._last_batch = sampler, batch_size, last_batch
        self._prev = []

    def __iter__(self):
        batch, self._prev = self._prev, []
        for i in self._sampler:
            batch.append(i)
            if len(batch) == self._batch_size:
                yield batch
                batch = []
        if batch:
            if self._last_batch == "keep":
                yield batch
            elif self._last_batch == "rollover":
                self._prev = batch

    def __len__(self):
        n, b = len(self._sampler), self._batch_size
        if self._last_batch == "keep":
            return (n + b - 1) // b
        if self._last_batch == "discard":
            return n // b
        return (len(self._prev) + n) // b

    def shuffle(self):
        self._sampler.shuffle()


class SliceSampler(Sampler):
    def __init__(self, length=None, indices=None, shuffle=False, seed=None):
        self.indices = list(range(length)) if indices is None else list(indices)
        self._rng = random.Random(seed)
        if shuffle:
            self.shuffle()

    def __iter__(self):
        return iter(self.indices)

    def __len__(self):
        return len(self.indices)

    def __getitem__(self, idx):
        if isinstance(idx, slice):
            return SliceSampler(indices=self.indices[idx])
        return self.indices[idx]

    def shuffle(self):
        self._rng.shuffle(self.indices)


class SliceBatchSampler(BatchSampler):
    def shuffle(self):
        self._sampler.shuffle()

    def __getitem__(self, idx):
        """Batches ``idx`` (a slice) of this sampler as a new batch sampler."""
        batches = list(iter(self))[idx]
        flat = [i for b in batches for i in b]
        return SliceBatchSampler(SliceSampler(indices=flat), self._batch_size, self._last_batch)
