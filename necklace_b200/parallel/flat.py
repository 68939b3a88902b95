"""Flat parameter / gradient storage.

All parameters of a module (or of one ``net_map`` unit) are re-pointed at slices
of one flat buffer and their gradients at slices of a second one, so that
collectives and optimizers see one contiguous range instead of a list of tensors.
This is the job of the reference's flat-memory manager
(necklace/frmwrk/pytorch/tsmem.py:30-79, :112-151, :157-217); differences: the
buffers can live in the symmetric peer-memory heap, shared (tied) parameters are
stored once, every slice starts on a 16-byte boundary (TMA / vector access), and
gradient kernels write straight into the flat gradient buffer (``_nkb_grad``
protocol of ``ops.gemm._deliver_grad``) so there is no flatten / unflatten copy
(reference: ptprms.py:256-299 flattens, reduces, unflattens and copies back).
"""
from __future__ import annotations

from typing import Callable, Iterable

import torch
import torch.nn as nn

ALIGN_ELEMS = 8  # 16 bytes of bf16


def _align(x: int, a: int) -> int:
    return (x + a - 1) // a * a


class FlatParams:
    def __init__(self, params: Iterable[nn.Parameter] | nn.Module, *,
                 alloc: Callable[[int, torch.dtype], torch.Tensor] | None = None,
                 pad_multiple: int = ALIGN_ELEMS, direct_grads: bool = True,
                 grad_dtype: torch.dtype | None = None):
        if isinstance(params, nn.Module):
            named = list(params.named_parameters())  # de-duplicates tied parameters
        else:
            named = [(f"p{i}", p) for i, p in enumerate(params)]
        seen, plist, names = set(), [], []
        for n, p in named:
            if p.requires_grad and id(p) not in seen:
                seen.add(id(p))
                plist.append(p)
                names.append(n)
        assert plist, "no trainable parameters"
        self.params, self.names = plist, names
        self.dtype = plist[0].dtype
        self.device = plist[0].device
        assert all(p.dtype == self.dtype for p in plist), "mixed parameter dtypes"
        self.offsets, off = [], 0
        for p in plist:
            self.offsets.append(off)
            off = _align(off + p.numel(), ALIGN_ELEMS)
        self.numel_used = off
        self.numel = _align(off, max(pad_multiple, ALIGN_ELEMS))
        gdt = grad_dtype or self.dtype
        if alloc is None:
            alloc = lambda n, dt: torch.zeros(n, dtype=dt, device=self.device)
        self.flat = alloc(self.numel, self.dtype)
        self.grad = alloc(self.numel, gdt)
        self.flat.zero_()
        self.grad.zero_()
        self.direct_grads = direct_grads
        for p, o in zip(plist, self.offsets):
            view = self.flat[o:o + p.numel()].view(p.shape)
            view.copy_(p.data)
            p.data = view
            gview = self.grad[o:o + p.numel()].view(p.shape)
            if direct_grads and gdt == self.dtype:
                p._nkb_grad = gview
                p._nkb_grad_has = False
            else:
                p.grad = gview
        self._unused_checked = False

    # gradient bookkeeping -------------------------------------------------
    def begin_step(self) -> None:
        """Mark all direct gradients as absent: the first kernel that produces a
        gradient overwrites its slice, later ones accumulate."""
        if self.direct_grads:
            for p in self.params:
                p._nkb_grad_has = False

    def finish_backward(self) -> None:
        """Fold gradients that autograd delivered the ordinary way (operators
        without direct delivery) into the flat buffer and zero slices that received
        nothing."""
        if not self.direct_grads:
            return
        for p, o in zip(self.params, self.offsets):
            g = p.grad
            if g is not None:
                if p._nkb_grad_has:
                    p._nkb_grad.add_(g)
                else:
                    p._nkb_grad.copy_(g)
                    p._nkb_grad_has = True
                p.grad = None
            elif not p._nkb_grad_has:
                p._nkb_grad.zero_()

    def zero_grad(self) -> None:
        self.grad.zero_()
        self.begin_step()

    def set_ready_callback(self, cb) -> None:
        for p in self.params:
            p._nkb_grad_ready = cb

    # views ------------------------------------------------------------------
    def grad_view(self, p: nn.Parameter) -> torch.Tensor:
        i = next(i for i, q in enumerate(self.params) if q is p)
        o = self.offsets[i]
        return self.grad[o:o + p.numel()].view(p.shape)

    def state_dict_flat(self) -> dict:
        return {"names": self.names, "offsets": self.offsets, "numel": self.numel}


class HeapGradReducer:
    """Data-parallel gradient reduction for an ordinary ``nn.Module`` + ``torch.optim``
    optimizer (the trainer API of the reference) on the fused peer-memory kernels.

    The module's parameters and ``.grad`` tensors are re-pointed at two flat buffers in the
    symmetric heap.  The gradient buffer is cut into buckets from its end; a
    post-accumulate-grad hook per parameter counts a bucket down and, when its last gradient
    has been written, launches the bucket's collective on a side stream (capped CTA count),
    so it runs under the rest of backward.  The collective is the fused 2-bit kernel
    (quantise + error feedback + exchange + decode, ``grad_comp_cfg`` as in the reference's
    ``grad_comp_threshold`` / ``grad_size_threshold`` keys) or the plain peer all-reduce, both
    with the 1/world scale folded in.  ``finish()`` launches what is left and joins the stream;
    the optimizer then steps on the reduced ``.grad`` views.

    Replaces flatten -> NCCL all-reduce -> divide -> unflatten -> copy after the whole backward
    (necklace/frmwrk/pytorch/ptprms.py:256-299)."""

    def __init__(self, module: nn.Module, peer, heap, grad_comp_cfg: dict | None = None,
                 bucket_mb: float = 25.0, overlap: bool = True, average: bool = True,
                 comm_ctas: int = 32):
        self.peer, self.world = peer, peer.world
        q = 8 * self.world * 64
        self.flat = FlatParams(module, alloc=lambda n, dt: heap.alloc(n, dt), pad_multiple=q,
                               direct_grads=False)
        f = self.flat
        self.scale = (1.0 / self.world) if average else 1.0
        self.cfg = grad_comp_cfg
        n = f.numel
        esz = f.grad.element_size()
        per = max(q, int(bucket_mb * (1 << 20) / esz) // q * q)
        self.buckets, hi = [], n
        while hi > 0:
            lo = max(0, hi - per)
            if lo < per // 2:
                lo = 0
            self.buckets.append((lo, hi))
            hi = lo
        self.compress = bool(grad_comp_cfg) and n >= int(grad_comp_cfg.get("grad_size_threshold", 0))
        if self.compress:
            self.thr = float(grad_comp_cfg.get("grad_comp_threshold", 0.5))
            self.residual = torch.zeros(n, dtype=torch.float32, device=f.device)
            self.codes = heap.alloc((n + 15) // 16, torch.int32)
            self.counts = heap.alloc((n + 15) // 16 * 16, torch.int8)
        # parameters per bucket (a parameter that straddles a boundary belongs to both)
        self._members = [[i for i, (p, o) in enumerate(zip(f.params, f.offsets))
                          if o < hi and o + p.numel() > lo] for lo, hi in self.buckets]
        self._of_param = {}
        for b, mem in enumerate(self._members):
            for i in mem:
                self._of_param.setdefault(i, []).append(b)
        self.overlap = overlap and len(self.buckets) > 1 and f.device.type == "cuda"
        self.comm_ctas = comm_ctas
        self._stream = torch.cuda.Stream(device=f.device, priority=-1) if self.overlap else None
        self._left, self._fired = [], set()
        if self.overlap:
            for i, p in enumerate(f.params):
                p.register_post_accumulate_grad_hook(self._make_hook(i))
        self.begin_backward()

    def _make_hook(self, i):
        def hook(_p):
            for b in self._of_param.get(i, ()):
                self._left[b] -= 1      # (a second backward of the same step goes negative)
                if self._left[b] == 0:
                    self._launch(b, side=True)
        return hook

    def begin_backward(self):
        self._left = [len(m) for m in self._members]
        self._fired = set()

    def _work(self, b, ctas):
        lo, hi = self.buckets[b]
        g = self.flat.grad[lo:hi]
        if self.compress:
            self.peer.dp_quant_allreduce(g, self.residual[lo:hi], self.codes[lo // 16:hi // 16],
                                         self.counts[lo:hi], g, self.thr, self.scale,
                                         max_ctas=ctas)
        else:
            self.peer.all_reduce(g, scale=self.scale, max_ctas=ctas)

    def _launch(self, b, side):
        if b in self._fired:
            return
        self._fired.add(b)
        if side and self._stream is not None:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            self._stream.wait_event(ev)
            with torch.cuda.stream(self._stream):
                self._work(b, self.comm_ctas)
        else:
            self._work(b, None)

    def finish(self):
        """Reduce every bucket that has not been launched yet and wait for the side stream
        (stream-ordered: the caller's stream continues after all buckets are done)."""
        for b in range(len(self.buckets)):
            self._launch(b, side=self._stream is not None)
        if self._stream is not None:
            ev = torch.cuda.Event()
            ev.record(self._stream)
            torch.cuda.current_stream().wait_event(ev)
        self.begin_backward()
