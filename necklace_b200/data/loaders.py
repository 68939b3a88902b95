"""Multi-process data loaders.

Two designs, both with ``num_workers`` daemon processes that each own every
``num_workers``-th batch of the epoch so that batch order is deterministic:

``QueueDataLoader``    workers collate batches and put them on one bounded queue per
                       worker; the consumer round-robins the queues
                       (reference: necklace/data/dtqpto.py:25-375, dtqptp.py).
``ShmRingDataLoader``  every worker owns a ring of ``part_num`` batch slots in shared
                       memory (torch CPU tensors in shared storage); it fills free
                       slots in place and posts the slot number, the consumer reads
                       the slot views and hands the slot back
                       (reference: necklace/data/dtmptp.py, dtmptv.py:27-533).

Both take an optional ``device``: batches are then copied from pinned staging
buffers to the GPU on a side stream one batch ahead of the consumer, so the
host-to-device copy overlaps the training step.
"""
from __future__ import annotations

import queue as pyqueue

import torch
import torch.multiprocessing as mp

from .batchify import stack_batchify_fn
from .sampler import BatchSampler, SliceBatchSampler, SliceSampler

_STOP, _EPOCH, _FREE = "stop", "epoch", "free"


def _batches_for(worker, num_workers, batches):
    return [b for i, b in enumerate(batches) if i % num_workers == worker]


def _queue_worker(dataset, collate, q_ctl, q_data):
    torch.set_num_threads(1)
    while True:
        msg = q_ctl.get()
        if msg[0] == _STOP:
            return
        if msg[0] == _EPOCH:
            for batch in msg[1]:
                try:
                    q_data.put(("batch", collate([dataset[i] for i in batch])))
                except Exception as e:  # noqa: BLE001
                    q_data.put(("error", repr(e)))
                    break
            q_data.put(("end", None))


def _ring_worker(dataset, collate, q_ctl, q_msg, slots, part_num):
    torch.set_num_threads(1)
    free = list(range(part_num))
    pending = []
    while True:
        msg = q_ctl.get()
        if msg[0] == _STOP:
            return
        if msg[0] == _FREE:
            free.append(msg[1])
            continue
        if msg[0] != _EPOCH:
            continue
        pending = list(msg[1])
        free = list(range(part_num))
        for batch in pending:
            while not free:
                m = q_ctl.get()
                if m[0] == _STOP:
                    return
                if m[0] == _FREE:
                    free.append(m[1])
            slot = free.pop(0)
            try:
                items = collate([dataset[i] for i in batch])
                items = items if isinstance(items, (tuple, list)) else (items,)
                n = items[0].shape[0]
                for ring, t in zip(slots, items):
                    ring[slot, :n].copy_(t)
                q_msg.put(("batch", slot, n))
            except Exception as e:  # noqa: BLE001
                q_msg.put(("error", repr(e), 0))
                break
        q_msg.put(("end", -1, 0))


class _LoaderBase:
    _attr_ngn_dataloader = True

    def __init__(self, dataset, batch_size=None, data_shape=None, shuffle=False, sampler=None,
                 last_batch=None, batch_sampler=None, batchify_fn=None, inter_batchify_fn=None,
                 part_num=4, num_workers=1, device=None, seed=None, timeout=120.0):
        """Argument order and names of the reference's loaders (necklace/data/dtqpto.py:31-38:
        ``dataset, batch_size, data_shape, shuffle, sampler, last_batch, batch_sampler,
        batchify_fn, inter_batchify_fn, part_num, num_workers``); ``data_shape`` (shape of one
        data item) is only needed by the shared-tensor ring, which can also infer it;
        ``num_workers=0`` (the reference's default) means one loader process."""
        if num_workers < 0:
            raise ValueError("num_workers should be >= 0")
        num_workers = max(1, int(num_workers))
        self.data_shape = tuple(data_shape) if data_shape is not None else None
        self.dataset, self.batch_size, self.shuffle = dataset, batch_size, shuffle
        self.last_batch = last_batch or "discard"
        self.batchify_fn = batchify_fn
        self.collate = inter_batchify_fn or stack_batchify_fn
        self.part_num, self.num_workers, self.timeout = part_num, num_workers, timeout
        self.device = torch.device(device) if device is not None else None
        if batch_sampler is None:
            if sampler is None:
                sampler = SliceSampler(len(dataset), shuffle=False, seed=seed)
            batch_sampler = self._make_batch_sampler(sampler)
        self.batch_sampler = batch_sampler
        self._ctx = mp.get_context("spawn")
        self._procs = []
        self._started = False

    def _make_batch_sampler(self, smplr):
        cls = SliceBatchSampler if isinstance(smplr, SliceSampler) else BatchSampler
        return cls(smplr, self.batch_size, self.last_batch)

    def reset_batch_sampler(self, new_sampler, *args, **kwargs):
        self.batch_sampler = self._make_batch_sampler(new_sampler)

    def __len__(self):
        return len(self.batch_sampler)

    def _epoch_batches(self):
        if self.shuffle:
            self.batch_sampler.shuffle()
        return list(self.batch_sampler)

    def _finish(self, items):
        """Optional user batchify + optional asynchronous copy to the device."""
        if self.batchify_fn is not None:
            items = self.batchify_fn(items)
        return items

    def _to_device_iter(self, it):
        if self.device is None or self.device.type != "cuda":
            yield from it
            return
        stream = torch.cuda.Stream(self.device)
        prev = None
        for items in it:
            with torch.cuda.stream(stream):
                cur = tuple(t.pin_memory().to(self.device, non_blocking=True)
                            if isinstance(t, torch.Tensor) else t for t in items)
                ev = torch.cuda.Event()
                ev.record(stream)
            if prev is not None:
                torch.cuda.current_stream(self.device).wait_event(prev[1])
                yield prev[0]
            prev = (cur, ev)
        if prev is not None:
            torch.cuda.current_stream(self.device).wait_event(prev[1])
            yield prev[0]

    def clear(self):
        for q in getattr(self, "qs_ctl", []):
            try:
                q.put((_STOP,))
            except Exception:  # noqa: BLE001
                pass
        for p in self._procs:
            p.join(timeout=2)
            if p.is_alive():
                p.terminate()
        self._procs = []
        self._started = False

    def __del__(self):
        try:
            self.clear()
        except Exception:  # noqa: BLE001
            pass


class QueueDataLoader(_LoaderBase):
    def _start(self):
        self.qs_ctl = [self._ctx.Queue() for _ in range(self.num_workers)]
        self.qs_data = [self._ctx.Queue(self.part_num) for _ in range(self.num_workers)]
        for w in range(self.num_workers):
            p = self._ctx.Process(target=_queue_worker, daemon=True,
                                  args=(self.dataset, self.collate, self.qs_ctl[w], self.qs_data[w]))
            p.start()
            self._procs.append(p)
        self._started = True

    def _raw_iter(self):
        if not self._started:
            self._start()
        batches = self._epoch_batches()
        for w in range(self.num_workers):
            self.qs_ctl[w].put((_EPOCH, _batches_for(w, self.num_workers, batches)))
        live = [True] * self.num_workers
        w = 0
        while any(live):
            if live[w]:
                try:
                    kind, payload = self.qs_data[w].get(timeout=self.timeout)
                except pyqueue.Empty:
                    raise RuntimeError(f"data worker {w} produced nothing for {self.timeout}s")
                if kind == "end":
                    live[w] = False
                elif kind == "error":
                    raise RuntimeError(f"data worker {w} failed: {payload}")
                else:
                    yield self._finish(payload)
            w = (w + 1) % self.num_workers

    def __iter__(self):
        return self._to_device_iter(self._raw_iter())


class ShmRingDataLoader(_LoaderBase):
    """``data_shapes`` = list of ``(shape_without_batch, dtype)`` per tensor of a batch;
    inferred from the first sample when omitted."""

    def __init__(self, dataset, batch_size=None, data_shape=None, data_shapes=None, **kw):
        super().__init__(dataset, batch_size, data_shape=data_shape, **kw)
        if data_shapes is None:
            sample = self.collate([dataset[0]])
            sample = sample if isinstance(sample, (tuple, list)) else (sample,)
            data_shapes = [(tuple(t.shape[1:]), t.dtype) for t in sample]
        self.data_shapes = data_shapes

    def _start(self):
        self.qs_ctl = [self._ctx.Queue() for _ in range(self.num_workers)]
        self.qs_msg = [self._ctx.Queue() for _ in range(self.num_workers)]
        self.rings = []
        for w in range(self.num_workers):
            slots = [torch.zeros((self.part_num, self.batch_size, *shape), dtype=dt).share_memory_()
                     for shape, dt in self.data_shapes]
            self.rings.append(slots)
            p = self._ctx.Process(target=_ring_worker, daemon=True,
                                  args=(self.dataset, self.collate, self.qs_ctl[w], self.qs_msg[w],
                                        slots, self.part_num))
            p.start()
            self._procs.append(p)
        self._started = True

    def _raw_iter(self):
        if not self._started:
            self._start()
        batches = self._epoch_batches()
        for w in range(self.num_workers):
            self.qs_ctl[w].put((_EPOCH, _batches_for(w, self.num_workers, batches)))
        live = [True] * self.num_workers
        w = 0
        while any(live):
            if live[w]:
                try:
                    kind, slot, n = self.qs_msg[w].get(timeout=self.timeout)
                except pyqueue.Empty:
                    raise RuntimeError(f"data worker {w} produced nothing for {self.timeout}s")
                if kind == "end":
                    live[w] = False
                elif kind == "error":
                    raise RuntimeError(f"data worker {w} failed: {slot}")
                else:
                    # copy out of the ring so the slot can be refilled while the
                    # consumer still uses the batch
                    items = tuple(ring[slot, :n].clone() for ring in self.rings[w])
                    self.qs_ctl[w].put((_FREE, slot))
                    yield self._finish(items)
            w = (w + 1) % self.num_workers

    def __iter__(self):
        return self._to_device_iter(self._raw_iter())


def _object_ring_worker(dataset, collate, q_ctl, q_msg, ring_name, slot_bytes, part_num):
    from .shmem import SharedMemArray
    ring = SharedMemArray(ring_name, slot_bytes, part_num)
    free = list(range(part_num))
    while True:
        msg = q_ctl.get()
        if msg[0] == _STOP:
            ring.close()
            return
        if msg[0] == _FREE:
            free.append(msg[1])
            continue
        if msg[0] != _EPOCH:
            continue
        free = list(range(part_num))
        for batch in msg[1]:
            while not free:
                m = q_ctl.get()
                if m[0] == _STOP:
                    ring.close()
                    return
                if m[0] == _FREE:
                    free.append(m[1])
            slot = free.pop(0)
            try:
                ring[slot] = collate([dataset[i] for i in batch])
                q_msg.put(("batch", slot, 0))
            except Exception as e:  # noqa: BLE001
                q_msg.put(("error", repr(e), 0))
                break
        q_msg.put(("end", -1, 0))


def _samples_as_they_are(samples):
    return samples


class ShmObjectRingDataLoader(_LoaderBase):
    """Ring of pickled batches in POSIX shared memory: a batch may be any picklable object
    (nested lists, dicts, numpy arrays, variable shapes), up to ``slot_bytes`` per batch.
    This is the design of the reference's ``dtmem`` / ``dtshm`` / ``dtshmp`` loaders
    (necklace/data/dtmem.py:19-396 over necklace/data/shmem.py); the default collate function
    here returns the list of samples unchanged."""

    def __init__(self, dataset, batch_size=None, data_shape=None, slot_bytes: int = 1 << 20, **kw):
        kw.setdefault("inter_batchify_fn", _samples_as_they_are)
        super().__init__(dataset, batch_size, data_shape=data_shape, **kw)
        self.slot_bytes = int(slot_bytes)

    def _start(self):
        from .shmem import SharedMemArray
        self.qs_ctl = [self._ctx.Queue() for _ in range(self.num_workers)]
        self.qs_msg = [self._ctx.Queue() for _ in range(self.num_workers)]
        self.rings = []
        for w in range(self.num_workers):
            ring = SharedMemArray(None, self.slot_bytes, self.part_num)
            self.rings.append(ring)
            p = self._ctx.Process(target=_object_ring_worker, daemon=True,
                                  args=(self.dataset, self.collate, self.qs_ctl[w], self.qs_msg[w],
                                        ring.name, self.slot_bytes, self.part_num))
            p.start()
            self._procs.append(p)
        self._started = True

    def _raw_iter(self):
        if not self._started:
            self._start()
        batches = self._epoch_batches()
        for w in range(self.num_workers):
            self.qs_ctl[w].put((_EPOCH, _batches_for(w, self.num_workers, batches)))
        live = [True] * self.num_workers
        w = 0
        while any(live):
            if live[w]:
                try:
                    kind, slot, _ = self.qs_msg[w].get(timeout=self.timeout)
                except pyqueue.Empty:
                    raise RuntimeError(f"data worker {w} produced nothing for {self.timeout}s")
                if kind == "end":
                    live[w] = False
                elif kind == "error":
                    raise RuntimeError(f"data worker {w} failed: {slot}")
                else:
                    item = self.rings[w][slot]
                    self.qs_ctl[w].put((_FREE, slot))
                    yield self._finish(item)
            w = (w + 1) % self.num_workers

    def __iter__(self):
        return self._raw_iter()

    def clear(self):
        super().clear()
        for ring in getattr(self, "rings", []):
            ring.close()
            ring.unlink()
        self.rings = []


# the class name every loader module of the reference exports
DataLoaderSharedMemory = ShmRingDataLoader
