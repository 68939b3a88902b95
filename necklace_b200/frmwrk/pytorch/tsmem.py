"""Flat-buffer memory manager for ZeRO (reference: necklace/frmwrk/pytorch/tsmem.py:30-217).

``md_params_to_flatten_1d_mem`` / ``md_grads_to_flatten_1d_mem`` re-point every
parameter (gradient) of a module at consecutive slices of one 1-D tensor.
``PtCudaFltnMemManager`` keeps one device weight buffer and one device gradient buffer
sized for the largest sub-module plus one host (pinned) buffer pair per sub-module, and
moves a sub-module between them by re-pointing, so a broadcast / reduce of a whole
sub-module is one collective on one flat range.  ``FlatParams`` (parallel/flat.py) is
the persistent-on-device variant the fused ZeRO kernel uses."""
from __future__ import annotations

import torch


def md_flatten_1d_mem_create(total_size, dtype=torch.float, device=torch.device("cpu"),
                             pin=False):
    t = torch.zeros(int(total_size), dtype=dtype, device=device)
    if pin and t.device.type == "cpu" and torch.cuda.is_available():
        t = t.pin_memory()
    return t


def md_flatten_1d_mem_reset(fltn):
    fltn.zero_()


def md_flatten_1d_mem_copy(frm_fltn, to_fltn, sz=-1):
    n = frm_fltn.numel() if sz is None or sz < 0 else sz
    to_fltn[:n].copy_(frm_fltn[:n], non_blocking=True)


def md_params_numel_total_size(md):
    return sum(p.numel() for p in md.parameters())


def md_grads_numel_total_size(md):
    return sum(p.numel() for p in md.parameters() if p.requires_grad)


def md_params_to_flatten_1d_mem(md, prm_fltn):
    """Copy the parameters into ``prm_fltn`` and make them views of it."""
    off = 0
    for p in md.parameters():
        n = p.numel()
        view = prm_fltn.narrow(0, off, n).view_as(p.data)
        view.copy_(p.data)
        p.data = view
        off += n
    return off


def md_grads_to_flatten_1d_mem(md, grd_fltn):
    off = 0
    for p in md.parameters():
        if not p.requires_grad:
            continue
        n = p.numel()
        view = grd_fltn.narrow(0, off, n).view_as(p.data)
        if p.grad is not None:
            view.copy_(p.grad.data)
        else:
            view.zero_()
        p.grad = view
        off += n
    return off


def md_params_to_flatten_1d_new(md, device):
    n = md_params_numel_total_size(md)
    dt = next(md.parameters()).dtype
    fl = md_flatten_1d_mem_create(n, dt, device)
    md_params_to_flatten_1d_mem(md, fl)
    return fl


def md_grads_to_flatten_1d_new(md, device):
    n = md_grads_numel_total_size(md)
    dt = next(md.parameters()).dtype
    fl = md_flatten_1d_mem_create(n, dt, device)
    md_grads_to_flatten_1d_mem(md, fl)
    return fl


class PtCudaFltnMemManager:
    def __init__(self, max_weig_size, max_grad_size, device, dtype=torch.float):
        self.device, self.dtype = torch.device(device), dtype
        self.gpu_weig = md_flatten_1d_mem_create(max_weig_size, dtype, self.device)
        self.gpu_grad = md_flatten_1d_mem_create(max_grad_size, dtype, self.device)
        self.cpu = {}  # id(module) -> (weights, grads, n_w, n_g)
        self.on_gpu = None      # id of the module currently living in the device buffers
        self.on_gpu_md = None

    def register(self, md):
        nw, ng = md_params_numel_total_size(md), md_grads_numel_total_size(md)
        w = md_flatten_1d_mem_create(nw, self.dtype, "cpu", pin=True)
        g = md_flatten_1d_mem_create(ng, self.dtype, "cpu", pin=True)
        md_params_to_flatten_1d_mem(md, w)
        md_grads_to_flatten_1d_mem(md, g)
        self.cpu[id(md)] = (w, g, nw, ng)

    def md_to_cpu(self, md):
        if id(md) not in self.cpu:
            self.register(md)
            return
        w, g, nw, ng = self.cpu[id(md)]
        if self.on_gpu == id(md):
            md_flatten_1d_mem_copy(self.gpu_weig, w, nw)
            md_flatten_1d_mem_copy(self.gpu_grad, g, ng)
            if self.device.type == "cuda":
                torch.cuda.current_stream().synchronize()
            self.on_gpu = self.on_gpu_md = None
        md_params_to_flatten_1d_mem(md, w)
        md_grads_to_flatten_1d_mem(md, g)

    def md_to_gpu(self, md):
        if self.on_gpu == id(md):
            return  # already resident: its device gradients must not be overwritten
        if self.on_gpu_md is not None:
            self.md_to_cpu(self.on_gpu_md)  # save the resident module first
        if id(md) not in self.cpu:
            self.register(md)
        w, g, nw, ng = self.cpu[id(md)]
        md_flatten_1d_mem_copy(w, self.gpu_weig, nw)
        md_flatten_1d_mem_copy(g, self.gpu_grad, ng)
        off = 0
        for p in md.parameters():
            n = p.numel()
            p.data = self.gpu_weig.narrow(0, off, n).view_as(p.data)
            off += n
        off = 0
        for p in md.parameters():
            if p.requires_grad:
                n = p.numel()
                p.grad = self.gpu_grad.narrow(0, off, n).view(p.data.shape)
                off += n
        self.on_gpu, self.on_gpu_md = id(md), md

    def weights_flat(self, md):
        return self.gpu_weig[:self.cpu[id(md)][2]]

    def grads_flat(self, md):
        return self.gpu_grad[:self.cpu[id(md)][3]]

    def zero_grad(self, md=None):
        self.gpu_grad.zero_()
        if md is not None and id(md) in self.cpu:
            self.cpu[id(md)][1].zero_()
