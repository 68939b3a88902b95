"""Symmetric peer-memory heap and the collectives that run on it.

``SymmetricHeap`` is one allocation per rank that every rank of the job maps
(through ``torch.distributed._symmetric_memory``: CUDA VMM handles exchanged over
the process group's store); ``PeerGroup`` is a subset of ranks with its own flag
region and epoch counter, on which the native kernels of ``csrc/comm.cu`` run:
barrier, all-reduce, all-gather, the 2-bit compressed gradient all-reduce and
the fused ZeRO step (reduce-scatter + optimizer + all-gather).

With one rank (or on CPU tensors, where ``TorchGroup`` stands in with
``torch.distributed`` collectives over gloo) the same calls degrade to their
local meaning, so trainers are written once.

This layer takes the place of the reference's pynccl communicator objects and
NCCL call wrappers (necklace/cuda/ncclgrp.py:24-60, necklace/cuda/ncclfns.py:65-260).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import _lib
from ..ops._common import status_word

_FLAG_REGION = 8192          # bytes reserved per group for epoch flags (160 CTAs x 8 ranks)
_MAX_GROUPS = 32


def _align(x: int, a: int) -> int:
    return (x + a - 1) // a * a


class SymmetricHeap:
    """A bump-allocated symmetric buffer.  Allocation order must be identical on all ranks."""

    def __init__(self, nbytes: int, group=None, device=None):
        self.device = torch.device(device if device is not None else
                                   f"cuda:{torch.cuda.current_device()}")
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.group = group
        total = _align(nbytes, 4096) + _FLAG_REGION * _MAX_GROUPS
        self.nbytes = total
        if self.world == 1:
            self.buf = torch.zeros(total, dtype=torch.uint8, device=self.device)
            self.ptrs = [self.buf.data_ptr()]
            self._hdl = None
        else:
            import torch.distributed._symmetric_memory as symm_mem
            self.buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
            self.buf.zero_()
            pg = group if group is not None else dist.group.WORLD
            self._hdl = symm_mem.rendezvous(self.buf, pg)
            self.ptrs = [int(p) for p in self._hdl.buffer_ptrs]
            torch.cuda.synchronize()
            dist.barrier(group)
        self._top = _FLAG_REGION * _MAX_GROUPS
        self._n_groups = 0

    # ------------------------------------------------------------ allocation
    def alloc(self, numel: int, dtype: torch.dtype, align: int = 256) -> torch.Tensor:
        """A tensor view inside the heap (same offset on every rank)."""
        esz = torch.empty(0, dtype=dtype).element_size()
        off = _align(self._top, align)
        end = off + numel * esz
        if end > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: need {end} of {self.nbytes} bytes")
        self._top = end
        # Not a view of ``self.buf``: views share one autograd version counter, so an in-place
        # write to ANY heap tensor would invalidate every heap tensor that some autograd
        # function saved for backward (token ids, gathered activations).  A fresh tensor over
        # the same storage has a counter of its own.
        t = torch.empty(0, dtype=dtype, device=self.device)
        t.set_(self.buf.untyped_storage(), (self.buf.storage_offset() + off) // esz, (numel,))
        return t

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.buf.data_ptr()
        assert 0 <= off < self.nbytes, "tensor is not inside this heap"
        return off

    def peer_group(self, ranks: list[int] | None = None) -> "PeerGroup":
        """A group over ``ranks`` (heap ranks, sorted).  Every rank must create its
        groups in the same order, including groups it is not a member of."""
        slot = self._n_groups
        self._n_groups += 1
        assert slot < _MAX_GROUPS
        ranks = list(range(self.world)) if ranks is None else list(ranks)
        return PeerGroup(self, ranks, slot * _FLAG_REGION)


class PeerGroup:
    def __init__(self, heap: SymmetricHeap, ranks: list[int], flag_off: int):
        self.heap, self.ranks, self.flag_off = heap, ranks, flag_off
        self.world = len(ranks)
        self.member = heap.rank in ranks
        self.rank = ranks.index(heap.rank) if self.member else -1
        dev = heap.device
        self.ptrs_dev = torch.tensor([heap.ptrs[r] for r in ranks], dtype=torch.int64, device=dev)
        self.epoch = torch.zeros(4, dtype=torch.int32, device=dev)
        self.max_ctas = 148

    def _ctx(self):
        return (self.ptrs_dev.data_ptr(), self.flag_off)

    def _tail(self, max_ctas=None):
        return (self.rank, self.world, self.epoch.data_ptr(),
                status_word(self.heap.device).data_ptr(),
                int(max_ctas if max_ctas is not None else self.max_ctas), _lib.stream_ptr())

    def barrier(self):
        if self.world == 1:
            return
        _lib.call("nkb_comm_barrier", *self._ctx(), self.rank, self.world, self.epoch.data_ptr(),
                  status_word(self.heap.device).data_ptr(), _lib.stream_ptr())
        _lib.count_launch()

    def all_reduce(self, t: torch.Tensor, scale: float = 1.0, max_ctas=None):
        """In-place sum over the group of a heap tensor (bf16 or fp32), times ``scale``."""
        assert t.dtype in (torch.bfloat16, torch.float32) and t.is_contiguous()
        if self.world == 1:
            if scale != 1.0:
                t.mul_(scale)
            return t
        _lib.call("nkb_comm_allreduce", *self._ctx(), self.heap.offset_of(t), t.numel(),
                  int(t.dtype == torch.float32), float(scale), *self._tail(max_ctas))
        _lib.count_launch()
        return t

    def all_gather(self, full: torch.Tensor, max_ctas=None):
        """``full`` (heap tensor) is ``world`` equal shards; this rank's shard is valid on
        entry, all shards on exit."""
        if self.world == 1:
            return full
        nbytes = full.numel() * full.element_size()
        assert nbytes % (16 * self.world) == 0
        _lib.call("nkb_comm_allgather", *self._ctx(), self.heap.offset_of(full),
                  nbytes // self.world, *self._tail(max_ctas))
        _lib.count_launch()
        return full

    def reduce_scatter(self, full: torch.Tensor, out: torch.Tensor | None = None,
                       scale: float = 1.0, max_ctas=None) -> torch.Tensor:
        """``out`` = this rank's 1/world slice (along dim 0) of the sum over the group of the
        heap tensor ``full``; ``full`` itself is left untouched."""
        W = self.world
        n = full.numel()
        shape = (full.shape[0] // W,) + tuple(full.shape[1:])
        if out is None:
            out = torch.empty(shape, dtype=full.dtype, device=full.device)
        if W == 1:
            out.copy_(full if scale == 1.0 else full * scale)
            return out
        assert full.is_contiguous() and out.is_contiguous() and out.numel() * W == n
        assert n % (256 * W) == 0, "reduce_scatter needs numel % (256 * world) == 0"
        _lib.call("nkb_comm_reduce_scatter", *self._ctx(), self.heap.offset_of(full), n,
                  int(full.dtype == torch.float32), float(scale), out.data_ptr(),
                  *self._tail(max_ctas))
        _lib.count_launch()
        return out

    def broadcast(self, t: torch.Tensor, root: int = 0, max_ctas=None) -> torch.Tensor:
        """Heap tensor ``t`` of the group's rank ``root`` is copied to every member's ``t``."""
        if self.world == 1:
            return t
        nbytes = t.numel() * t.element_size()
        assert t.is_contiguous() and nbytes % 16 == 0
        _lib.call("nkb_comm_bcast", *self._ctx(), self.heap.offset_of(t), nbytes, int(root),
                  *self._tail(max_ctas))
        _lib.count_launch()
        return t

    def dp_quant_allreduce(self, g, residual, codes, counts, out, thr, scale, max_ctas=None):
        """Fused 2-bit compressed all-reduce; ``codes`` / ``counts`` are heap tensors."""
        n = g.numel()
        _lib.call("nkb_comm_dp_quant_allreduce", *self._ctx(), g.data_ptr(),
                  int(g.dtype == torch.float32), residual.data_ptr(), self.heap.offset_of(codes),
                  self.heap.offset_of(counts), out.data_ptr(), int(out.dtype == torch.float32), n,
                  float(thr), float(scale), *self._tail(max_ctas))
        _lib.count_launch()
        return out

    def rs_opt_ag(self, grads, params, master, s1, s2, *, adam: bool, lr, beta1=0.9, beta2=0.999,
                  eps=1e-8, weight_decay=0.0, step=1, grad_scale=1.0, first_step=False,
                  max_ctas=None, hyper=None):
        """Fused ZeRO step on heap tensors ``grads`` / ``params`` (bf16, full length)."""
        n = grads.numel()
        c1 = 1.0 / (1.0 - beta1 ** step) if adam else 1.0
        c2 = 1.0 / (1.0 - beta2 ** step) if adam else 1.0
        _lib.call("nkb_comm_rs_opt_ag", *self._ctx(), self.heap.offset_of(grads),
                  self.heap.offset_of(params), n, master.data_ptr(),
                  s1.data_ptr() if s1 is not None else None,
                  s2.data_ptr() if s2 is not None else None, int(adam), float(lr), float(beta1),
                  float(beta2), float(eps), float(weight_decay), float(c1), float(c2),
                  float(grad_scale), int(first_step),
                  hyper.data_ptr() if hyper is not None else None, *self._tail(max_ctas))
        _lib.count_launch()


    @staticmethod
    def _auto_ag_ctas(world: int, M: int, N: int, K: int) -> int:
        """Copy CTAs for the fused all-gather: the fewest (even, 4..32) whose push of this
        rank's shard to all peers ends before the GEMM on the remaining SMs does.  Rates: a
        copy CTA moved ~19 GB/s of posted stores over NVLink, the GEMM ~1.3 PFLOP/s on 148
        SMs (both measured on B200)."""
        nbytes = (world - 1) * (M // world) * K * 2
        flops = 2.0 * M * N * K
        for c in range(4, 32, 2):
            t_copy = nbytes / (c * 19e9)
            t_gemm = flops / (1.3e15 * (148 - c) / 148)
            if t_copy <= 0.85 * t_gemm:
                return c
        return 32

    def ag_gemm(self, x_full: torch.Tensor, w: torch.Tensor, *, out=None, bias=None, b_mn=False,
                ag_ctas: int = 0, bn: int = 0) -> torch.Tensor:
        """``out = all_gather_rows(x) @ w^T`` in one kernel.  ``x_full`` is a heap tensor
        ``[world * R, K]`` whose rows ``[rank*R, (rank+1)*R)`` hold this rank's shard; the
        other rows are filled by the peers' copy CTAs (each rank pushes its shard to every
        peer with posted stores) while the GEMM CTAs already work on the local rows."""
        from ..ops._common import ptr
        M, K = x_full.shape
        R = M // self.world
        N = w.shape[1] if b_mn else w.shape[0]
        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=x_full.device)
        if ag_ctas <= 0:
            ag_ctas = self._auto_ag_ctas(self.world, M, N, K)
        nblk = self.world * ((R + 127) // 128)
        flags = getattr(self, "_ag_flags", None)
        if flags is None or flags.numel() < nblk:
            # in the heap (peers raise the flags), at the same offset on every member: all
            # members make the same calls in the same order.  Fresh heap memory is zero.
            flags = self.heap.alloc(max(nblk, 4096), torch.int32)
            self._ag_flags = flags
        _lib.call("nkb_ag_gemm_bf16", self.ptrs_dev.data_ptr(), self.flag_off,
                  self.heap.offset_of(x_full), self.rank, self.world, R, self.epoch.data_ptr(),
                  flags.data_ptr(), int(ag_ctas), x_full.stride(0), w.data_ptr(), w.stride(0),
                  int(b_mn), out.data_ptr(), out.stride(0), int(out.dtype == torch.float32), N, K,
                  ptr(bias), None, 0, 0, None, 0, x_full.data_ptr(),
                  status_word(self.heap.device).data_ptr(), int(bn), _lib.stream_ptr())
        _lib.count_launch()
        return out


    def gemm_rs(self, x: torch.Tensor, w: torch.Tensor, *, out=None, bias=None, res=None,
                b_mn=False, bn: int = 0) -> torch.Tensor:
        """``out[R, N]`` = this rank's row block of ``sum_ranks x_r @ w_r^T`` (+ bias + res):
        GEMM and reduce-scatter in one kernel.  ``x``: ``[M, K_local]`` with ``M = world*R``;
        partial tiles of other ranks' rows are stored directly into the owner's staging slab
        over NVLink (bf16); the epilogue of an own tile adds the peers' partial tiles to its
        fp32 accumulator as their flags arrive."""
        from ..ops._common import ptr
        M, K = x.shape
        N = w.shape[1] if b_mn else w.shape[0]
        R = M // self.world
        key = (R, N)
        cache = getattr(self, "_rs_cache", None)
        if cache is None:
            cache = self._rs_cache = {}
        if key not in cache:
            stage = self.heap.alloc(self.world * R * N, torch.bfloat16)
            tflags = self.heap.alloc(self.world * (R // 128) * ((N + 127) // 128), torch.int32)
            # No zeroing here: the heap is zero-filled before it is mapped and the bump
            # allocator never hands a range out twice.  Zeroing now would race with a
            # faster peer whose kernel is already raising flags in this rank's array.
            cache[key] = (stage, tflags)
        stage, tflags = cache[key]
        if out is None:
            out = torch.empty(R, N, dtype=torch.bfloat16, device=x.device)
        _lib.call("nkb_gemm_rs_bf16", self.ptrs_dev.data_ptr(), self.flag_off,
                  self.heap.offset_of(stage), self.heap.offset_of(tflags), self.rank, self.world,
                  R, self.epoch.data_ptr(), x.data_ptr(), x.stride(0), w.data_ptr(),
                  w.stride(0), int(b_mn), out.data_ptr(), out.stride(0), N, K, ptr(bias), ptr(res),
                  res.stride(0) if res is not None else 0,
                  status_word(self.heap.device).data_ptr(), int(bn), _lib.stream_ptr())
        _lib.count_launch()
        return out


class TorchGroup:
    """Same surface as ``PeerGroup`` on top of ``torch.distributed`` collectives
    (gloo on CPU, NCCL on GPU).  It is the CPU test double and the NCCL baseline."""

    def __init__(self, group=None, ranks: list[int] | None = None):
        self.group = group
        if dist.is_initialized():
            self.world = dist.get_world_size(group)
            self.rank = dist.get_rank(group)
        else:
            self.world, self.rank = 1, 0
        self.ranks = ranks if ranks is not None else list(range(self.world))
        self.member = self.rank >= 0

    def barrier(self):
        if self.world > 1:
            dist.barrier(self.group)

    def all_reduce(self, t, scale: float = 1.0, max_ctas=None):
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        if scale != 1.0:
            t.mul_(scale)
        return t

    def all_gather(self, full, max_ctas=None):
        if self.world > 1:
            shard = full.view(self.world, -1)[self.rank].clone()
            dist.all_gather_into_tensor(full.view(-1), shard, group=self.group)
        return full

    def reduce_scatter(self, full, out=None, scale: float = 1.0, max_ctas=None):
        W = self.world
        shape = (full.shape[0] // W,) + tuple(full.shape[1:])
        if out is None:
            out = torch.empty(shape, dtype=full.dtype, device=full.device)
        if W == 1:
            out.copy_(full)
        else:
            acc = full.float().contiguous()   # gloo has no reduce-scatter: reduce all, keep mine
            dist.all_reduce(acc, group=self.group)
            per = full.shape[0] // W
            out.copy_(acc[self.rank * per:(self.rank + 1) * per].to(out.dtype))
        if scale != 1.0:
            out.mul_(scale)
        return out

    def broadcast(self, t, root: int = 0, max_ctas=None):
        if self.world > 1:
            dist.broadcast(t, src=self.ranks[root] if self.group is not None else root,
                           group=self.group)
        return t

    def dp_quant_allreduce(self, g, residual, codes, counts, out, thr, scale, max_ctas=None):
        from ..ops.quant import quantize_flat
        n = g.numel()
        quantize_flat(g.reshape(-1), residual, thr, codes)
        # decode locally to ternary, sum over ranks (what the fused kernel does with counts)
        from ..ops.quant import dequantize_flat
        tern = torch.empty(n, dtype=torch.float32, device=g.device)
        dequantize_flat(codes, tern, 1.0)
        if self.world > 1:
            dist.all_reduce(tern, group=self.group)
        out.reshape(-1).copy_((tern * (thr * scale)).to(out.dtype))
        return out

    def ag_gemm(self, x_full, w, *, out=None, bias=None, b_mn=False, ag_ctas=8, bn=0):
        """Unfused stand-in of ``PeerGroup.ag_gemm``: all-gather the rows, then the GEMM."""
        from ..ops.gemm import gemm
        if self.world > 1:
            R = x_full.shape[0] // self.world
            mine = x_full[self.rank * R:(self.rank + 1) * R].clone()
            dist.all_gather_into_tensor(x_full, mine, group=self.group)
        return gemm(x_full, w, b_mn=b_mn, bias=bias, out=out)

    def gemm_rs(self, x, w, *, out=None, bias=None, res=None, b_mn=False, bn=0):
        """Unfused stand-in of ``PeerGroup.gemm_rs``: GEMM (fp32 out), reduce-scatter of the
        rows, then bias and residual."""
        from ..ops.gemm import gemm
        part = gemm(x, w, b_mn=b_mn, out_dtype=torch.float32)
        mine = self.reduce_scatter(part)
        if bias is not None:
            mine = mine + bias.float()
        if res is not None:
            mine = mine + res.float()
        mine = mine.to(x.dtype)
        if out is not None:
            out.copy_(mine)
            return out
        return mine

    def rs_opt_ag(self, grads, params, master, s1, s2, *, adam, lr, beta1=0.9, beta2=0.999,
                  eps=1e-8, weight_decay=0.0, step=1, grad_scale=1.0, first_step=False,
                  max_ctas=None, hyper=None):
        from ..ops.optim import adam_step, sgd_step
        n = grads.numel()
        shard = n // self.world
        g32 = grads.float()
        if self.world > 1:
            dist.all_reduce(g32, group=self.group)
        mine = g32[self.rank * shard:(self.rank + 1) * shard].contiguous()
        pshard = params[self.rank * shard:(self.rank + 1) * shard]
        if adam:
            adam_step(master, s1, s2, mine, pshard, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                      weight_decay=weight_decay, step=step, grad_scale=grad_scale, hyper=hyper)
        else:
            sgd_step(master, s1, mine, pshard, lr=lr, momentum=beta1, weight_decay=weight_decay,
                     first_step=first_step, grad_scale=grad_scale, hyper=hyper)
        self.all_gather(params)
