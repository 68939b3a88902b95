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
