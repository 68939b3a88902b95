"""Whole-step engine for pipeline-parallel training (``dp+pp`` and ``dp+pp+mp``).

A ``PipelineEngine`` owns one pipeline stage.  One call to ``step`` runs all micro-batches
of a global step through the one-forward-one-backward schedule, then the data-parallel
gradient reduction and the optimizer of ``TrainEngine`` (peer-memory all-reduce kernels,
bucketed and overlapped with the last micro-batch's backward when ``bucket_mb`` is set).

The reference runs one batch through the stages strictly one after the other and relays
every tensor shape through the scheduler on every transfer (necklace/trainer/ppoppt.py:277-329,
necklace/trainer/tndspp.py:1202-1291).  Here:

* shapes are negotiated once: the very first transfer of a channel carries a header, both
  sides cache it, every later transfer is the bare payload (no host synchronisation in the
  steady state);
* receives are posted ahead: the receive of micro-batch k+1 (or of the next gradient) is
  issued before the compute that precedes its use, so the NCCL transfer overlaps the kernels;
* the two directions of a stage pair use different communicators, so a posted receive never
  queues in front of a send going the other way;
* with tensor parallelism inside a stage only this rank's ``[tokens/p, C]`` rows travel
  (the residual stream is row-sharded), i.e. 1/p of the reference's bytes.
"""
from __future__ import annotations

from collections import deque

import torch
import torch.distributed as dist

from . import pipeline as P
from .engine import TrainEngine

_HDR = 32


class _Chan:
    """One direction of a stage pair with cached payload shapes."""

    def __init__(self, src: int, dst: int, device):
        self.src, self.dst, self.device = src, dst, device
        self.group = P._chan(src, dst)
        self.specs = None           # [(shape, dtype)] once negotiated
        self.keep = []              # sent tensors and their works, until flushed

    # sender ---------------------------------------------------------------
    def send(self, tensors):
        tensors = [t.detach().contiguous() for t in tensors]
        if self.specs is None:
            hdr = torch.zeros(_HDR, dtype=torch.int64)
            hdr[0] = len(tensors)
            k = 1
            for t in tensors:
                hdr[k], hdr[k + 1] = P._DTYPES.index(t.dtype), t.dim()
                for j, s in enumerate(t.shape):
                    hdr[k + 2 + j] = s
                k += 2 + t.dim()
            hdr = hdr.to(P._hdr_device(self.device))
            self.keep.append((dist.isend(hdr, self.dst, group=self.group), hdr))
            self.specs = [(tuple(t.shape), t.dtype) for t in tensors]
        else:
            got = [(tuple(t.shape), t.dtype) for t in tensors]
            if got != self.specs:
                raise RuntimeError(f"pipeline payload changed from {self.specs} to {got}; "
                                   "micro-batch shapes must stay fixed")
        for t in tensors:
            self.keep.append((dist.isend(t, self.dst, group=self.group), t))

    def flush(self):
        for w, _ in self.keep:
            w.wait()
        self.keep = []

    # receiver ---------------------------------------------------------------
    def post_recv(self):
        """Issue the receives of one payload; returns a handle for ``wait_recv``."""
        if self.specs is None:
            dev = P._hdr_device(self.device)
            hdr = torch.zeros(_HDR, dtype=torch.int64, device=dev)
            dist.irecv(hdr, self.src, group=self.group).wait()
            hdr = hdr.cpu()         # the only host synchronisation of this channel, once
            specs, k = [], 1
            for _ in range(int(hdr[0])):
                dt, nd = P._DTYPES[int(hdr[k])], int(hdr[k + 1])
                specs.append((tuple(int(x) for x in hdr[k + 2:k + 2 + nd]), dt))
                k += 2 + nd
            self.specs = specs
        bufs = [torch.empty(s, dtype=d, device=self.device) for s, d in self.specs]
        works = [dist.irecv(b, self.src, group=self.group) for b in bufs]
        return works, bufs

    @staticmethod
    def wait_recv(handle):
        works, bufs = handle
        for w in works:
            w.wait()
        return bufs


class PipelineEngine(TrainEngine):
    """``model``: this stage's module.  First stage: ``model(tokens)`` -> activation(s);
    middle: ``model(*acts)`` -> activation(s); last: ``model(*acts, targets)`` -> scalar loss
    (a single-stage pipeline calls ``model(tokens, targets)``).  ``pp_ranks``: global ranks of
    this pipeline group in stage order.  ``group`` / ``heap``: the data-parallel peer group and
    the symmetric heap (as for ``TrainEngine``); ``micro_batches``: micro-batches per step."""

    def __init__(self, model, *, stage: int, pp_ranks: list[int], micro_batches: int = 1,
                 group=None, heap=None, mp_group=None, prepost: bool = True, **kw):
        mode = kw.pop("mode", None) or ("dp" if group is not None and group.world > 1 else "local")
        kw.pop("use_cuda_graph", None)   # NCCL p2p inside the step: launched eagerly
        super().__init__(model, mode=mode, group=group, heap=heap, micro_batches=micro_batches,
                         use_cuda_graph=False, **kw)
        self.stage, self.pp_ranks = stage, list(pp_ranks)
        self.n_stage = len(pp_ranks)
        self.first, self.last = stage == 0, stage == self.n_stage - 1
        self.mp_group = mp_group
        self.prepost = prepost     # issue receives one transfer ahead of their use
        dev = self.flat.device
        me = pp_ranks[stage]
        self.fwd_in = None if self.first else _Chan(pp_ranks[stage - 1], me, dev)
        self.fwd_out = None if self.last else _Chan(me, pp_ranks[stage + 1], dev)
        self.bwd_in = None if self.last else _Chan(pp_ranks[stage + 1], me, dev)
        self.bwd_out = None if self.first else _Chan(me, pp_ranks[stage - 1], dev)
        self._bcast_buf = {}

    # input broadcast over the tensor-parallel group ------------------------------------
    def broadcast_inputs(self, *tensors, root: int = 0):
        """The tensor-parallel group's rank ``root`` holds the batch; every member gets it
        (peer-memory broadcast kernel; the reference broadcasts shape and data over NCCL every
        step, necklace/trainer/tnoppt.py:285-317).  Shapes must be known on all members."""
        g = self.mp_group
        if g is None or g.world == 1:
            return tensors
        out = []
        for i, t in enumerate(tensors):
            key = (i, tuple(t.shape), t.dtype)
            buf = self._bcast_buf.get(key)
            if buf is None:
                n = (t.numel() * t.element_size() + 15) // 16 * 16 // t.element_size()
                buf = g.heap.alloc(n, t.dtype)
                self._bcast_buf[key] = buf
            view = buf[:t.numel()].view(t.shape)
            if g.rank == root:
                view.copy_(t, non_blocking=True)
            g.broadcast(buf, root)
            out.append(view)
        return tuple(out)

    # one micro-batch -----------------------------------------------------------------
    def _forward_mb(self, x, y, recv_handle):
        if self.first:
            inputs, tgt = [x], y
        else:
            got = _Chan.wait_recv(recv_handle)
            inputs, tgt = got[:-1], got[-1]
            inputs = [t.requires_grad_(True) if t.is_floating_point() else t for t in inputs]
        if self.last:
            loss = self.model(*inputs, tgt)
            self._inflight.append((inputs, [loss]))
            self._losses.append(loss.detach())
        else:
            out = self.model(*inputs)
            outs = list(out) if isinstance(out, (tuple, list)) else [out]
            self.fwd_out.send(outs + [tgt])
            self._inflight.append((inputs, outs))

    def _backward_mb(self, recv_handle):
        inputs, outs = self._inflight.popleft()
        if self.last:
            outs[0].backward()
        else:
            grads = _Chan.wait_recv(recv_handle)
            fouts = [o for o in outs if o.is_floating_point()]   # one gradient per float output
            pairs = [(o, g) for o, g in zip(fouts, grads) if o.requires_grad]
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        if not self.first:
            gin = [t.grad if t.grad is not None else torch.zeros_like(t)
                   for t in inputs if t.is_floating_point()]
            self.bwd_out.send(gin)

    # the schedule ---------------------------------------------------------------------
    def _fwd_bwd(self, x=None, y=None):
        m = self.micro_batches
        self.flat.begin_step()
        self._inflight, self._losses = deque(), []
        if self.first:
            xs, ys = x.chunk(m, dim=0), y.chunk(m, dim=0)
        warm = min(self.n_stage - self.stage - 1, m)
        fwd = bwd = 0
        nxt_f = self.fwd_in.post_recv() if not self.first else None
        nxt_b = None

        def run_fwd():
            nonlocal fwd, nxt_f
            h = nxt_f
            nxt_f = None
            if not self.first and h is None:
                h = self.fwd_in.post_recv()
            if self.first:
                self._forward_mb(xs[fwd], ys[fwd], None)
            else:
                got_ready = h
                # post the next micro-batch's receive before computing this one
                if fwd + 1 < m and self.prepost:
                    nxt_f = self.fwd_in.post_recv()
                self._forward_mb(None, None, got_ready)
            fwd += 1

        def run_bwd():
            nonlocal bwd, nxt_b
            h = nxt_b
            nxt_b = None
            if not self.last and h is None:
                h = self.bwd_in.post_recv()
            self._armed = bwd == m - 1          # overlap buckets under the last backward
            self._backward_mb(h)
            self._armed = False
            bwd += 1

        for _ in range(warm):
            run_fwd()
        while fwd < m:
            # the gradient of the oldest micro-batch in flight arrives while we compute (not
            # before the channel's first transfer: its header can only come after our forward)
            if not self.last and self.prepost and self.bwd_in.specs is not None:
                nxt_b = self.bwd_in.post_recv()
            run_fwd()
            run_bwd()
        while bwd < m:
            run_bwd()
        for ch in (self.fwd_out, self.bwd_out):
            if ch is not None:
                ch.flush()
        self.flat.finish_backward()
        if self.last:
            return torch.stack(self._losses).mean()
        return torch.zeros((), device=self.flat.device)
