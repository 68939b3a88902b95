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

With ``use_cuda_graph`` the whole step (forward, backward, collective,
optimizer) is captured once and replayed; the per-step scalars that change
(learning rate, Adam bias corrections) live in a small device tensor.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from ..ops import adam_step, sgd_step
from ..ops._common import check_status
from .flat import FlatParams


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
                 use_cuda_graph: bool = False, grad_average: bool = True):
        assert mode in ("local", "dp", "zero")
        self.model, self.mode, self.group, self.heap = model, mode, group, heap
        self.optim = optim or OptimConfig()
        self.grad_comp = grad_comp
        self.world = group.world if group is not None else 1
        self.rank = group.rank if group is not None else 0
        self.grad_scale = (1.0 / self.world) if grad_average else 1.0
        alloc = None
        if heap is not None and self.world > 1:
            alloc = lambda n, dt: heap.alloc(n, dt)
        self.flat = FlatParams(model, alloc=alloc, pad_multiple=8 * self.world * 64)
        dev = self.flat.device
        n = self.flat.numel
        self.sharded = mode == "zero" and self.world > 1
        nstate = n // self.world if self.sharded else n
        lo = self.rank * nstate if self.sharded else 0
        self.master = self.flat.flat[lo:lo + nstate].float()
        self.s1 = torch.zeros(nstate, dtype=torch.float32, device=dev)
        self.s2 = torch.zeros(nstate, dtype=torch.float32, device=dev) \
            if self.optim.kind == "adam" else None
        if self.optim.kind == "sgd" and self.optim.beta1 == 0.0:
            self.s1 = None
        self.step_count = 0
        self.hyper = torch.zeros(4, dtype=torch.float32, device=dev)
        self._hyper_host = torch.zeros(4, dtype=torch.float32,
                                       pin_memory=dev.type == "cuda")
        if grad_comp is not None and mode == "dp":
            self.residual = torch.zeros(n, dtype=torch.float32, device=dev)
            nwords = (n + 15) // 16
            if alloc is not None:
                self.codes = heap.alloc(nwords, torch.int32)
                self.counts = heap.alloc(nwords * 16, torch.int8)
            else:
                self.codes = torch.zeros(nwords, dtype=torch.int32, device=dev)
                self.counts = torch.zeros(nwords * 16, dtype=torch.int8, device=dev)
        self.use_cuda_graph = use_cuda_graph and dev.type == "cuda"
        self._graph = None
        self._static_in = None
        self._static_loss = None

    # ----------------------------------------------------------- one step
    def _set_hyper(self) -> None:
        o = self.optim
        t = self.step_count
        self._hyper_host[0] = o.lr
        if o.kind == "adam":
            self._hyper_host[1] = 1.0 / (1.0 - math.pow(o.beta1, t))
            self._hyper_host[2] = 1.0 / (1.0 - math.pow(o.beta2, t))
        self.hyper.copy_(self._hyper_host, non_blocking=True)

    def _fwd_bwd(self, *inputs):
        self.flat.begin_step()
        loss = self.model(*inputs)
        loss.backward()
        self.flat.finish_backward()
        return loss.detach()

    def _reduce_and_update(self) -> None:
        o, f = self.optim, self.flat
        first = self.step_count == 1
        if self.sharded:
            self.group.rs_opt_ag(f.grad, f.flat, self.master, self.s1, self.s2,
                                 adam=o.kind == "adam", lr=o.lr, beta1=o.beta1, beta2=o.beta2,
                                 eps=o.eps, weight_decay=o.weight_decay, step=self.step_count,
                                 grad_scale=self.grad_scale, first_step=first,
                                 hyper=self.hyper if o.kind == "adam" else None)
            return
        gscale = 1.0
        if self.mode == "dp" and self.world > 1:
            if self.grad_comp is not None and f.numel >= self.grad_comp.grad_size_threshold:
                self.group.dp_quant_allreduce(f.grad, self.residual, self.codes, self.counts,
                                              f.grad, self.grad_comp.grad_comp_threshold,
                                              self.grad_scale)
            else:
                self.group.all_reduce(f.grad, scale=self.grad_scale)
        elif self.mode == "dp" and self.grad_comp is not None and self.group is not None:
            # single rank: the codec still runs so the numerics match the multi-rank path
            self.group.dp_quant_allreduce(f.grad, self.residual, self.codes, self.counts, f.grad,
                                          self.grad_comp.grad_comp_threshold, 1.0)
        if o.kind == "adam":
            adam_step(self.master, self.s1, self.s2, f.grad, f.flat, lr=o.lr, beta1=o.beta1,
                      beta2=o.beta2, eps=o.eps, weight_decay=o.weight_decay,
                      step=self.step_count, grad_scale=gscale, hyper=self.hyper)
        else:
            sgd_step(self.master, self.s1, f.grad, f.flat, lr=o.lr, momentum=o.beta1,
                     weight_decay=o.weight_decay, first_step=first, grad_scale=gscale)

    def _eager_step(self, *inputs):
        loss = self._fwd_bwd(*inputs)
        self._reduce_and_update()
        return loss

    def step(self, *inputs) -> torch.Tensor:
        """Run one optimizer step; returns the (device) loss of this rank's batch."""
        self.step_count += 1
        self._set_hyper()
        if not self.use_cuda_graph:
            return self._eager_step(*inputs)
        if self._graph is None:
            return self._capture(*inputs)
        for s, x in zip(self._static_in, inputs):
            s.copy_(x, non_blocking=True)
        self._graph.replay()
        return self._static_loss

    def _capture(self, *inputs):
        # SGD's first step differs from the rest (momentum initialisation), and kernels
        # configure their shared-memory limits on first use: run eagerly once, then capture.
        loss = self._eager_step(*inputs)
        if self.optim.kind == "sgd" and self.step_count == 1:
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
        if not self.sharded:
            return self.master.clone()
        import torch.distributed as dist
        parts = [torch.empty_like(self.master) for _ in range(self.world)]
        dist.all_gather(parts, self.master)
        return torch.cat(parts)
