"""Fused flat-buffer optimizers (Adam/AdamW, SGD-momentum) and flat helpers.

State lives in flat fp32 buffers (master weights, first/second moments or the
momentum buffer); gradients are read from a flat bf16/fp32 buffer and the updated
weights are also written as bf16 into the flat parameter buffer the model
computes with.  One kernel per optimizer step per flat buffer replaces the
per-parameter ``opt.step()`` loop of the reference trainers
(necklace/trainer/tnoppt.py:493-498).
"""
from __future__ import annotations

import math

import torch

from .. import _lib
from ._common import on_gpu, ptr


def adam_step(master, m, v, grad, param_bf16, *, lr, beta1=0.9, beta2=0.999, eps=1e-8,
              weight_decay=0.0, step=1, grad_scale=1.0, hyper=None):
    """One Adam(W) step over flat buffers.  ``step`` is 1-based.  ``hyper`` is an optional
    device tensor ``[lr, 1/(1-b1^t), 1/(1-b2^t), t, gmul]`` (see ``hyper_advance``) that
    overrides the host values of lr and the bias corrections and multiplies ``grad_scale``
    by ``gmul``, so a CUDA graph can be replayed with a changing step count."""
    n = master.numel()
    c1 = 1.0 / (1.0 - beta1 ** step)
    c2 = 1.0 / (1.0 - beta2 ** step)
    if not on_gpu(master):
        if hyper is not None:
            lr, c1, c2 = (float(x) for x in hyper[:3])
            grad_scale = grad_scale * float(hyper[4])
        g = grad.float() * grad_scale
        m.mul_(beta1).add_(g, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        upd = (m * c1) / ((v * c2).sqrt() + eps)
        master.sub_(lr * (upd + weight_decay * master))
        if param_bf16 is not None:
            param_bf16.copy_(master.to(param_bf16.dtype))
        return
    assert master.dtype == torch.float32 and m.dtype == torch.float32 and v.dtype == torch.float32
    assert grad.dtype in (torch.bfloat16, torch.float32) and grad.numel() == n
    _lib.call("nkb_adam_flat", master.data_ptr(), m.data_ptr(), v.data_ptr(), grad.data_ptr(),
              int(grad.dtype == torch.float32), ptr(param_bf16), n, float(lr), float(beta1),
              float(beta2), float(eps), float(weight_decay), float(c1), float(c2),
              float(grad_scale), ptr(hyper), _lib.stream_ptr())
    _lib.count_launch()


def sgd_step(master, mom, grad, param_bf16, *, lr, momentum=0.0, weight_decay=0.0,
             first_step=False, grad_scale=1.0, hyper=None):
    n = master.numel()
    if not on_gpu(master):
        if hyper is not None:
            lr = float(hyper[0])
            grad_scale = grad_scale * float(hyper[4])
        g = grad.float() * grad_scale + weight_decay * master
        if mom is not None:
            if first_step:
                mom.copy_(g)
            else:
                mom.mul_(momentum).add_(g)
            g = mom
        master.sub_(lr * g)
        if param_bf16 is not None:
            param_bf16.copy_(master.to(param_bf16.dtype))
        return
    _lib.call("nkb_sgd_flat", master.data_ptr(), ptr(mom), grad.data_ptr(),
              int(grad.dtype == torch.float32), ptr(param_bf16), n, float(lr), float(momentum),
              float(weight_decay), float(grad_scale), int(first_step), ptr(hyper),
              _lib.stream_ptr())
    _lib.count_launch()


def scale_cast(src, dst, scale=1.0, accumulate=False):
    """dst = (dst if accumulate else 0) + scale * src over flat bf16/fp32 buffers."""
    n = src.numel()
    assert dst.numel() == n
    if not on_gpu(src, dst):
        val = src.float() * scale
        dst.copy_(((dst.float() + val) if accumulate else val).to(dst.dtype))
        return dst
    _lib.call("nkb_scale_cast", src.data_ptr(), int(src.dtype == torch.float32), dst.data_ptr(),
              int(dst.dtype == torch.float32), n, float(scale), int(accumulate),
              _lib.stream_ptr())
    _lib.count_launch()
    return dst


def sumsq(src, out=None):
    """Adds sum(src^2) into ``out`` (fp32 scalar tensor); used for gradient-norm clipping."""
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=src.device)
    if not on_gpu(src):
        out += src.float().pow(2).sum()
        return out
    _lib.call("nkb_sumsq", src.data_ptr(), int(src.dtype == torch.float32), src.numel(),
              out.data_ptr(), _lib.stream_ptr())
    _lib.count_launch()
    return out


def hyper_advance(hyper, beta1, beta2):
    """``hyper = [lr, c1, c2, t, gmul, ...]`` (fp32, on the optimizer's device): ``t += 1`` and
    the Adam bias corrections ``c1 = 1/(1-beta1^t)``, ``c2 = 1/(1-beta2^t)`` are recomputed from
    it.  The step count lives on the device so that the values used by step ``t`` do not
    depend on how far the host has run ahead."""
    if not on_gpu(hyper):
        t = float(hyper[3]) + 1.0
        hyper[3] = t
        hyper[1] = 1.0 / (1.0 - math.pow(beta1, t))
        hyper[2] = 1.0 / (1.0 - math.pow(beta2, t))
        return hyper
    _lib.call("nkb_hyper_advance", hyper.data_ptr(), float(beta1), float(beta2),
              _lib.stream_ptr())
    _lib.count_launch()
    return hyper


def clip_coef(hyper, sumsq_t, max_norm, grad_scale=1.0):
    """``hyper[4] = min(1, max_norm / (sqrt(sumsq) * grad_scale))``, on the device."""
    if not on_gpu(hyper):
        nrm = float(sumsq_t.sqrt()) * grad_scale
        hyper[4] = min(1.0, max_norm / (nrm + 1e-6))
        hyper[5] = nrm
        return hyper
    _lib.call("nkb_clip_coef", hyper.data_ptr(), sumsq_t.data_ptr(), float(max_norm),
              float(grad_scale), _lib.stream_ptr())
    _lib.count_launch()
    return hyper


def bias_corrections(beta1, beta2, step):
    return 1.0 / (1.0 - math.pow(beta1, step)), 1.0 / (1.0 - math.pow(beta2, step))
