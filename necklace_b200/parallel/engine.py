"""Whole-step training engine for the data-parallel and ZeRO modes.

One call to ``TrainEngine.step`` runs forward, backward, the gradient
collective and the optimizer of one global step inside the worker process,
with no control-plane round trip (the reference's scheduler drives every phase
by RPC and synchronises the device around each NCCL call:
necklace/trainer/tndsnc.py:687-710, necklace/trainer/tnoppt.py:540-554).

Modes:
  ``local``  single rank: fused flat optimizer.
  ``dp``     gradient all-reduce over the group (optionally the fused 2-bit
             compressed all-reduce with error feedback), then the fused flat
             optimizer on fp32 master weights.
  ``zero``   ZeRO: one fused kernel does the gradient reduce-scatter, the
             optimizer on this rank's fp32 shard and the all-gather of the new
             bf16 parameters into every rank's parameter buffer.

Gradient accumulation: ``micro_batches=k`` splits every input along dim 0 into
``k`` chunks; their gradients accumulate in the flat gradient buffer and the
collective + optimizer run once.

Overlap: with ``bucket_mb`` set, the flat buffer is cut into buckets from its end
(backward produces the last parameters' gradients first).  As soon as the last
gradient kernel of a bucket has been enqueued, the bucket's collective (and, where
no global quantity is needed, its optimizer update) is launched on a side stream
with a capped CTA count, so it runs under the rest of the backward pass.  The
reference reduces one 256 MB bucket after another only after the whole backward
(necklace/frmwrk/pytorch/ptprms.py:256-299).

With ``use_cuda_graph`` the whole step (all micro-batches, both streams) is
captured once and replayed.  The scalars that change per step (Adam bias
corrections, clipping coefficient) are computed on the device from a device step
counter, so neither graph replay nor a host that runs ahead of the device can
pair a step with another step's scalars.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import adam_step, sgd_step
from ..ops._common import check_status
from ..ops.optim import clip_coef, hyper_advance, sumsq
from .flat import FlatParams

HYPER_LR, HYPER_C1, HYPER_C2, HYPER_T, HYPER_GMUL = 0, 1, 2, 3, 4


@dataclass
class OptimConfig:
    kind: str = "adam"          # "adam" | "sgd"
    lr: float = 1e-4
    beta1: float = 0.9          # Adam beta1 / SGD momentum
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0


@dataclass
class GradCompConfig:
    """2-bit gradient compression (keys follow the reference's ``grad_comp_cfg``:
    ``grad_comp_threshold`` is the quantisation threshold, tensors smaller than
    ``grad_size_threshold`` elements would be sent uncompressed; with one flat
    buffer the latter only switches compression off for tiny models)."""
    grad_comp_threshold: float = 0.5
    grad_size_threshold: int = 0


class TrainEngine:
    def __init__(self, model: torch.nn.Module, *, mode: str = "local", group=None, heap=None,
                 optim: OptimConfig | None = None, grad_comp: GradCompConfig | None = None,
                 use_cuda_graph: bool = False, grad_average: bool = True,
                 micro_batches: int = 1, bucket_mb: float | None = None, comm_ctas: int = 32,
                 clip_grad_norm: float | None = None, grad_sync=None):
        assert mode in ("local", "dp", "zero")
        self.model, self.mode, self.group, self.heap = model, mode, group, heap
        self.optim = optim or OptimConfig()
        self.grad_comp = grad_comp
        self.world = group.world if group is not None else 1
        self.rank = group.rank if group is not None else 0
        self.micro_batches = int(micro_batches)
        self.grad_scale = ((1.0 / self.world) if grad_average else 1.0) / self.micro_batches
        self.clip = clip_grad_norm
        self.comm_ctas = comm_ctas
        # optional callable run once per step after the last backward and before any bucket
        # that holds the parameters it touches is reduced (``grad_sync.params``): used for
        # gradients that another parallel dimension has to combine first
        self.grad_sync = grad_sync
        alloc = None
        if heap is not None and self.world > 1:
            alloc = lambda n, dt: heap.alloc(n, dt)
        self.quantum = 8 * self.world * 64
        self.flat = FlatParams(model, alloc=alloc, pad_multiple=self.quantum)
        dev = self.flat.device
        n = self.flat.numel
        self.sharded = mode == "zero" and self.world > 1
        self.buckets = self._make_buckets(bucket_mb)
        self.overlap = bucket_mb is not None and dev.type == "cuda"
        nstate = n // self.world if self.sharded else n
        self.master = self.shard_of(self.flat.flat.float())
        assert self.master.numel() == nstate
        self.s1 = torch.zeros(nstate, dtype=torch.float32, device=dev)
        self.s2 = torch.zeros(nstate, dtype=torch.float32, device=dev) \
            if self.optim.kind == "adam" else None
        if self.optim.kind == "sgd" and self.optim.beta1 == 0.0:
            self.s1 = None
        self.step_count = 0
        # device scalars {lr, 1/(1-b1^t), 1/(1-b2^t), t, gradient multiplier}
        self.hyper = torch.zeros(8, dtype=torch.float32, device=dev)
        self.hyper[HYPER_LR] = self.optim.lr
        self.hyper[HYPER_GMUL] = 1.0
        self.gnorm_sq = torch.zeros(1, dtype=torch.float32, device=dev) \
            if self.clip is not None else None
        if grad_comp is not None and mode == "dp":
            self.residual = torch.zeros(n, dtype=torch.float32, device=dev)
            nwords = (n + 15) // 16
            if heap is not None:
                self.codes = heap.alloc(nwords, torch.int32)
                self.counts = heap.alloc(nwords * 16, torch.int8)
            else:
                self.codes = torch.zeros(nwords, dtype=torch.int32, device=dev)
                self.counts = torch.zeros(nwords * 16, dtype=torch.int8, device=dev)
        self.use_cuda_graph = use_cuda_graph and dev.type == "cuda"
        self._graph = None
        self._static_in = None
        self._static_loss = None
        # overlap bookkeeping: learnt from the first step's gradient-delivery order
        self._order: list[int] | None = None      # parameter index per delivery
        self._fire_at: dict[int, list[int]] | None = None
        self._recording: list[int] | None = None
        # NKB_DEBUG_STREAMS=1: logical check that bucket work on the side stream and gradient
        # writes on the main stream are ordered by the events below (utils/streamcheck.py)
        from ..utils import streamcheck
        self._chk = streamcheck.from_env()
        self._deliveries = 0
        self._fired: set[int] = set()
        self._armed = False
        self._comm_stream = None
        self._pidx = {id(p): i for i, p in enumerate(self.flat.params)}
        if self.overlap and len(self.buckets) > 1:
            self._comm_stream = torch.cuda.Stream(device=dev, priority=-1)
            self.flat.set_ready_callback(self._on_grad_ready)

    # ----------------------------------------------------------- layout
    def _make_buckets(self, bucket_mb) -> list[tuple[int, int]]:
        """[lo, hi) element ranges, last range first (the order backward completes them)."""
        n, q = self.flat.numel, self.quantum
        if bucket_mb is None:
            return [(0, n)]
        per = max(q, int(bucket_mb * (1 << 20) / 2) // q * q)
        out, hi = [], n
        while hi > 0:
            lo = max(0, hi - per)
            if lo < per // 2:      # do not leave a sliver at the front
                lo = 0
            out.append((lo, hi))
            hi = lo
        return out

    def shard_of(self, full: torch.Tensor) -> torch.Tensor:
        """This rank's part of a flat full-length tensor: with ZeRO, slice ``rank`` of every
        bucket (stored at ``lo / world``); otherwise all of it."""
        if not self.sharded:
            return full.clone()
        W, r = self.world, self.rank
        out = torch.empty(full.numel() // W, dtype=full.dtype, device=full.device)
        for lo, hi in self.buckets:
            per = (hi - lo) // W
            out[lo // W:hi // W] = full[lo + r * per:lo + (r + 1) * per]
        return out

    def gather_state(self, shard: torch.Tensor, pg=None) -> torch.Tensor:
        """Inverse of ``shard_of`` (collective over the ZeRO ranks when sharded)."""
        if not self.sharded:
            return shard.clone()
        import torch.distributed as dist
        parts = [torch.empty_like(shard) for _ in range(self.world)]
        dist.all_gather(parts, shard.contiguous(), group=pg)
        full = torch.empty(shard.numel() * self.world, dtype=shard.dtype, device=shard.device)
        W = self.world
        for lo, hi in self.buckets:
            per = (hi - lo) // W
            for r in range(W):
                full[lo + r * per:lo + (r + 1) * per] = parts[r][lo // W:hi // W]
        return full

    # ----------------------------------------------------------- scalars
    def set_lr(self, lr: float) -> None:
        """Change the learning rate (stream-ordered: takes effect for steps enqueued later)."""
        self.optim.lr = float(lr)
        self.hyper[HYPER_LR:HYPER_LR + 1].fill_(float(lr))

    def set_step_count(self, t: int) -> None:
        self.step_count = int(t)
        self.hyper[HYPER_T:HYPER_T + 1].fill_(float(t))

    # ----------------------------------------------------------- overlap
    def _on_grad_ready(self, p) -> None:
        if not self._armed:
            return
        i = self._pidx.get(id(p))
        if i is None:
            return
        if self._recording is not None:
            self._recording.append(i)
            return
        k = self._deliveries
        self._deliveries += 1
        if self._chk is not None:
            for b in self._buckets_of(i):
                self._chk.access(f"bucket{b}", "main", True, f"gradient of parameter {i}")
        if self._order is None or k >= len(self._order) or self._order[k] != i:
            raise RuntimeError("gradient delivery order changed between steps; overlapped "
                               "buckets need a static model (construct with bucket_mb=None)")
        for b in self._fire_at.get(k, ()):
            self._launch_bucket(b, side=True)

    def _buckets_of(self, i: int) -> list[int]:
        """Buckets that hold a part of parameter ``i``."""
        o, n = self.flat.offsets[i], self.flat.params[i].numel()
        return [b for b, (lo, hi) in enumerate(self.buckets) if o < hi and o + n > lo]

    def _learn_order(self, seq: list[int]) -> None:
        f = self.flat
        last = {}
        for k, i in enumerate(seq):
            last[i] = k
        for p in getattr(self.grad_sync, "params", ()):   # their buckets wait for grad_sync
            last.pop(self._pidx.get(id(p)), None)
        fire: dict[int, list[int]] = {}
        for b, (lo, hi) in enumerate(self.buckets):
            need = -1
            for i, (p, o) in enumerate(zip(f.params, f.offsets)):
                if o < hi and o + p.numel() > lo:
                    if i not in last:       # gradient arrives through autograd: wait for the end
                        need = None
                        break
                    need = max(need, last[i])
            if need is not None and need >= 0:
                fire.setdefault(need, []).append(b)
        self._order, self._fire_at = seq, fire

    def _launch_bucket(self, b: int, side: bool) -> None:
        if b in self._fired:
            return
        self._fired.add(b)
        if side and self._comm_stream is not None:
            cur = torch.cuda.current_stream()
            ev = torch.cuda.Event()
            ev.record(cur)
            self._comm_stream.wait_event(ev)
            if self._chk is not None:
                self._chk.wait("side", self._chk.record("main"))
                self._chk.access(f"bucket{b}", "side", True, "bucket collective / update")
            with torch.cuda.stream(self._comm_stream):
                self._bucket_work(b, self.comm_ctas)
        else:
            if self._chk is not None:
                self._chk.access(f"bucket{b}", "main", True, "bucket collective / update")
            self._bucket_work(b, None)

    def _join_side(self) -> None:
        if self._comm_stream is not None:
            ev = torch.cuda.Event()
            ev.record(self._comm_stream)
            torch.cuda.current_stream().wait_event(ev)
            if self._chk is not None:
                self._chk.join("main", "side")

    # ----------------------------------------------------------- per-bucket work
    def _opt_range(self, lo: int, hi: int, grad, param, state_lo: int) -> None:
        o = self.optim
        n = hi - lo
        sl = slice(state_lo, state_lo + n)
        if o.kind == "adam":
            adam_step(self.master[sl], self.s1[sl], self.s2[sl], grad, param, lr=o.lr,
                      beta1=o.beta1, beta2=o.beta2, eps=o.eps, weight_decay=o.weight_decay,
                      step=max(self.step_count, 1), grad_scale=self._opt_gscale,
                      hyper=self.hyper)
        else:
            sgd_step(self.master[sl], self.s1[sl] if self.s1 is not None else None, grad, param,
                     lr=o.lr, momentum=o.beta1, weight_decay=o.weight_decay,
                     first_step=self.step_count == 1, grad_scale=self._opt_gscale,
                     hyper=self.hyper)

    def _bucket_work(self, b: int, ctas) -> None:
        """Collective (+ optimizer unless a global norm is needed first) of one bucket."""
        o, f = self.optim, self.flat
        lo, hi = self.buckets[b]
        g, p = f.grad[lo:hi], f.flat[lo:hi]
        W = self.world
        if self.sharded and self.clip is None:
            sl = slice(lo // W, hi // W)
            self.group.rs_opt_ag(g, p, self.master[sl], self.s1[sl] if self.s1 is not None else None,
                                 self.s2[sl] if self.s2 is not None else None,
                                 adam=o.kind == "adam", lr=o.lr, beta1=o.beta1, beta2=o.beta2,
                                 eps=o.eps, weight_decay=o.weight_decay,
                                 step=max(self.step_count, 1), grad_scale=self.grad_scale,
                                 first_step=self.step_count == 1, max_ctas=ctas,
                                 hyper=self.hyper)
            return
        reduced_scale = 1.0     # what is still to be applied to the gradient in the optimizer
        if W > 1 and self.mode in ("dp", "zero"):
            if self.mode == "dp" and self.grad_comp is not None and \
                    f.numel >= self.grad_comp.grad_size_threshold:
                wl, wh = lo // 16, hi // 16
                self.group.dp_quant_allreduce(g, self.residual[lo:hi], self.codes[wl:wh],
                                              self.counts[lo:hi], g,
                                              self.grad_comp.grad_comp_threshold,
                                              self.grad_scale, max_ctas=ctas)
            else:
                self.group.all_reduce(g, scale=self.grad_scale, max_ctas=ctas)
        elif self.mode == "dp" and self.grad_comp is not None and self.group is not None:
            # single rank: the codec still runs so the numerics match the multi-rank path
            self.group.dp_quant_allreduce(g, self.residual[lo:hi], self.codes[lo // 16:hi // 16],
                                          self.counts[lo:hi], g,
                                          self.grad_comp.grad_comp_threshold, self.grad_scale)
        else:
            reduced_scale = self.grad_scale
        self._opt_gscale = reduced_scale
        if self.clip is None:
            self._bucket_update(b)

    def _bucket_update(self, b: int) -> None:
        f, W = self.flat, self.world
        lo, hi = self.buckets[b]
        if self.sharded:      # clipped ZeRO: gradients were all-reduced; update my slice, gather
            per = (hi - lo) // W
            mlo = lo + self.rank * per
            self._opt_range(mlo, mlo + per, f.grad[mlo:mlo + per], f.flat[mlo:mlo + per], lo // W)
            self.group.all_gather(f.flat[lo:hi])
        else:
            self._opt_range(lo, hi, f.grad[lo:hi], f.flat[lo:hi], lo)

    # ----------------------------------------------------------- one step
    def _fwd_bwd(self, *inputs):
        k = self.micro_batches
        self.flat.begin_step()
        if k == 1:
            self._armed = True
            loss = self.model(*inputs)
            loss.backward()
            self._armed = False
            total = loss.detach()
        else:
            chunks = [x.chunk(k, dim=0) for x in inputs]
            total = None
            for j in range(k):
                self._armed = j == k - 1
                loss = self.model(*(c[j] for c in chunks))
                loss.backward()
                total = loss.detach() if total is None else total + loss.detach()
            self._armed = False
            total = total / k
        self.flat.finish_backward()
        return total

    def _eager_step(self, *inputs):
        o = self.optim
        if o.kind == "adam":
            hyper_advance(self.hyper, o.beta1, o.beta2)
        self._fired = set()
        self._deliveries = 0
        self._opt_gscale = self.grad_scale
        learn = self._comm_stream is not None and self._order is None
        self._recording = [] if learn else None
        loss = self._fwd_bwd(*inputs)
        if self.grad_sync is not None:
            self.grad_sync()
        side = self._comm_stream is not None and not learn
        for b in range(len(self.buckets)):
            self._launch_bucket(b, side=side)
        self._join_side()
        if learn:
            self._learn_order(self._recording)
            self._recording = None
        elif self._order is not None and self._deliveries != len(self._order):
            raise RuntimeError("fewer gradient deliveries than in the first step; overlapped "
                               "buckets need a static model (construct with bucket_mb=None)")
        if self.clip is not None:
            self._clipped_update()
        return loss

    def _clipped_update(self) -> None:
        """Global-norm clipping: every bucket's gradient is reduced by now; the coefficient
        min(1, max_norm / ||g||) is computed on the device and multiplies the gradient inside
        the optimizer kernels."""
        f = self.flat
        self.gnorm_sq.zero_()
        sumsq(f.grad, self.gnorm_sq)
        clip_coef(self.hyper, self.gnorm_sq, self.clip, self._opt_gscale)
        for b in range(len(self.buckets)):
            self._bucket_update(b)

    def step(self, *inputs) -> torch.Tensor:
        """Run one optimizer step; returns the (device) loss of this rank's batch."""
        self.step_count += 1
        if not self.use_cuda_graph:
            return self._eager_step(*inputs)
        if self._graph is None:
            return self._capture(*inputs)
        for s, x in zip(self._static_in, inputs):
            s.copy_(x, non_blocking=True)
        self._graph.replay()
        return self._static_loss

    def _capture(self, *inputs):
        # SGD's first step differs from the rest (momentum initialisation), kernels
        # configure their shared-memory limits on first use and the overlap schedule is
        # learnt from an eager step: run eagerly first, then capture.
        loss = self._eager_step(*inputs)
        if (self.optim.kind == "sgd" and self.step_count == 1) or \
                (self._comm_stream is not None and self.step_count == 1):
            return loss
        torch.cuda.synchronize()
        self._static_in = [x.clone() if x.is_cuda else x.to(self.flat.device) for x in inputs]
        g = torch.cuda.CUDAGraph()
        from .. import _lib
        l0 = _lib.launch_count
        with torch.cuda.graph(g):
            self._static_loss = self._eager_step(*self._static_in)
        self.launches_per_step = _lib.launch_count - l0  # native launches replayed per step
        self._graph = g  # capturing executes nothing; later calls replay
        return loss

    def check(self) -> None:
        """Synchronise and raise if any kernel reported a device-side error."""
        if self.flat.device.type == "cuda":
            check_status()

    # ------------------------------------------------------------ checkpoint
    def full_master(self) -> torch.Tensor:
        """fp32 master weights of the whole flat buffer (gathered when sharded)."""
        return self.gather_state(self.master)
