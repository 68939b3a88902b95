"""Pipeline parallelism: self-describing point-to-point transfers and a micro-batched
1F1B schedule that runs entirely inside the worker.

The reference pipeline is strictly sequential (one batch, one stage busy at a time) and
every transfer is set up by the scheduler, which also relays tensor shapes in RPC
payloads (necklace/trainer/tndspp.py:1202-1291, necklace/trainer/ppoppt.py:277-329).
Here a transfer carries its own header (count, dtypes, shapes), activations travel with
``torch.distributed`` p2p (NCCL on GPU) posted ahead of use, and a step is split into
``micro_batches`` that flow through the stages one-forward-one-backward, so that all
stages are busy in the steady state.  ``micro_batches=1`` reproduces the reference's
sequential behaviour.
"""
from __future__ import annotations

from collections import deque

import torch
import torch.distributed as dist

_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int64, torch.int32,
           torch.int16, torch.int8, torch.uint8, torch.bool]
_HDR = 64
END_MARK = -1


def _hdr_device(device):
    # NCCL needs device tensors; gloo takes CPU tensors
    return torch.device(device) if dist.get_backend() == "nccl" else torch.device("cpu")


# One-directional channels between neighbouring stages: (src, dst) -> process group.
# Activations (forward direction) and gradients (backward direction) of a stage pair
# use different communicators, so a stage that is sending its activation never queues
# behind, or in front of, the gradient its neighbour is sending the other way.
_CHANNELS: dict = {}
_PENDING: list = []


def create_channels(pp_groups) -> None:
    """Collective over the whole job: every rank calls this with the same list of
    pipeline groups (stage-ordered global ranks)."""
    for grp in pp_groups or []:
        for a, b in zip(grp[:-1], grp[1:]):
            for key in ((a, b), (b, a)):
                if key not in _CHANNELS:
                    _CHANNELS[key] = dist.new_group([a, b])


def _chan(src, dst):
    return _CHANNELS.get((src, dst))


def flush_sends() -> None:
    """Wait for every posted send (call before the buffers they read are reused)."""
    while _PENDING:
        w, _keep = _PENDING.pop()
        w.wait()


def p2p_send(tensors, dst: int, device=None, end: bool = False):
    """Post the send of a list of tensors (or of an end-of-epoch marker) to global rank
    ``dst``.  Returns at once; ``flush_sends`` waits for completion."""
    me = dist.get_rank()
    dev = _hdr_device(device if device is not None else (tensors[0].device if tensors else "cpu"))
    hdr = torch.zeros(_HDR, dtype=torch.int64)
    if end:
        hdr[0] = END_MARK
    else:
        hdr[0] = len(tensors)
        k = 1
        for t in tensors:
            hdr[k] = _DTYPES.index(t.dtype)
            hdr[k + 1] = t.dim()
            for j, sz in enumerate(t.shape):
                hdr[k + 2 + j] = sz
            k += 2 + t.dim()
            assert k <= _HDR, "too many / too high-rank tensors for one transfer header"
    grp = _chan(me, dst)
    payload = [hdr.to(dev)]
    if not end:
        payload += [t.detach().contiguous().to(dev) for t in tensors]
    for t in payload:
        _PENDING.append((dist.isend(t, dst, group=grp), t))


def p2p_recv(src: int, device):
    """Receive what ``p2p_send`` sent; returns a list of tensors or ``None`` for the marker."""
    me = dist.get_rank()
    dev = _hdr_device(device)
    grp = _chan(src, me)
    hdr = torch.zeros(_HDR, dtype=torch.int64, device=dev)
    dist.irecv(hdr, src, group=grp).wait()
    hdr = hdr.cpu()
    n = int(hdr[0])
    if n == END_MARK:
        return None
    out, k = [], 1
    for _ in range(n):
        dt, nd = _DTYPES[int(hdr[k])], int(hdr[k + 1])
        shape = [int(x) for x in hdr[k + 2:k + 2 + nd]]
        k += 2 + nd
        out.append(torch.empty(shape, dtype=dt, device=dev))
    works = [dist.irecv(t, src, group=grp) for t in out]
    for w in works:
        w.wait()
    return [t.to(device) for t in out]


class PipelineStage:
    """One stage of a pipeline group.

    ``net`` maps the stage inputs to its outputs; the last stage also owns ``loss_fn``.
    ``ranks`` are the global ranks of the pipeline group in stage order."""

    def __init__(self, net, stage: int, ranks: list[int], loss_fn=None, device="cpu"):
        self.net, self.stage, self.ranks = net, stage, ranks
        self.n_stage = len(ranks)
        self.loss_fn, self.device = loss_fn, torch.device(device)
        self.first, self.last = stage == 0, stage == len(ranks) - 1
        self.prev = ranks[stage - 1] if not self.first else None
        self.next = ranks[stage + 1] if not self.last else None
        self.inflight = deque()   # (inputs, outputs) of forwarded, not yet back-propagated mbs
        self.losses = []

    # one micro-batch ---------------------------------------------------------------
    def forward_mb(self, data=None, target=None):
        """Returns False when the epoch has ended (marker received / no data).  Targets
        travel down the pipeline next to the activations."""
        if self.first:
            if data is None:
                if self.n_stage > 1:
                    p2p_send([], self.next, self.device, end=True)
                return False
            inputs, tgt = [data.to(self.device)], target.to(self.device)
        else:
            got = p2p_recv(self.prev, self.device)
            if got is None:
                if not self.last:
                    p2p_send([], self.next, self.device, end=True)
                return False
            inputs, tgt = got[:-1], got[-1]
            inputs = [x.requires_grad_(True) if x.is_floating_point() else x for x in inputs]
        out = self.net(*inputs)
        outs = list(out) if isinstance(out, (tuple, list)) else [out]
        if self.last:
            loss = self.loss_fn(out, tgt)
            self.inflight.append((inputs, [loss]))
            self.losses.append(loss.detach())
        else:
            p2p_send([o.detach() for o in outs] + [tgt], self.next, self.device)
            self.inflight.append((inputs, outs))
        return True

    def backward_mb(self, scale: float = 1.0):
        inputs, outs = self.inflight.popleft()
        if self.last:
            (outs[0] * scale).backward()
        else:
            grads = p2p_recv(self.next, self.device)
            pairs = [(o, g) for o, g in zip(outs, grads) if o.requires_grad]
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        if not self.first:
            gin = [x.grad if (x.is_floating_point() and x.grad is not None) else
                   torch.zeros_like(x, dtype=torch.float32) for x in inputs]
            p2p_send(gin, self.prev, self.device)

    # one step = m micro-batches, 1F1B -------------------------------------------------
    def run_step(self, micro_batches):
        """``micro_batches``: list of ``(data, target)`` on the first stage (``None`` entries
        elsewhere), or ``None`` on the first stage when the epoch is over.  Returns the mean
        loss on the last stage, ``True`` on other stages, ``False`` at the end of the epoch."""
        m = len(micro_batches) if micro_batches is not None else 1
        if self.first and micro_batches is None:
            self.forward_mb(None, None)
            flush_sends()
            return False
        warm = min(self.n_stage - self.stage - 1, m)
        self.losses = []
        fwd = bwd = 0
        scale = 1.0 / m
        get = (lambda i: micro_batches[i]) if self.first else (lambda i: (None, None))
        for _ in range(warm):
            if not self.forward_mb(*get(fwd)):
                return False
            fwd += 1
        while fwd < m:
            if not self.forward_mb(*get(fwd)):
                return False
            fwd += 1
            self.backward_mb(scale)
            bwd += 1
        while bwd < fwd:
            self.backward_mb(scale)
            bwd += 1
        flush_sends()
        if self.last:
            return torch.stack(self.losses).mean()
        return True
