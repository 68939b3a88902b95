"""LayerNorm / RMSNorm with hand-written forward and backward kernels."""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import _lib
from ._common import on_gpu, ptr, scratch
from .gemm import _deliver_grad, colsum_scratch


def norm_fwd(x2: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None, eps: float, rms: bool):
    rows, Cn = x2.shape
    if not on_gpu(x2):
        xf = x2.float()
        mean = torch.zeros(rows, device=x2.device) if rms else xf.mean(1)
        var = ((xf - mean[:, None]) ** 2).mean(1)
        rstd = torch.rsqrt(var + eps)
        y = (xf - mean[:, None]) * rstd[:, None] * w.float()
        if b is not None:
            y = y + b.float()
        return y.to(x2.dtype), torch.stack([mean, rstd], 1)
    assert x2.dtype == torch.bfloat16 and x2.is_contiguous()
    y = torch.empty_like(x2)
    stats = torch.empty(rows, 2, dtype=torch.float32, device=x2.device)
    _lib.call("nkb_norm_fwd", x2.data_ptr(), w.data_ptr(), ptr(b), y.data_ptr(), stats.data_ptr(),
              rows, Cn, float(eps), int(rms), _lib.stream_ptr())
    _lib.count_launch()
    return y, stats


def norm_bwd(dy2, x2, w, stats, rms: bool, need_wgrad: bool = True, need_bgrad: bool = True,
             dres=None):
    """Returns (dx, dw_fp32 or None, db_fp32 or None); dw/db are fp32 rows of length C.
    ``dres`` (optional, same shape as x2) is added to dx inside the kernel: the gradient that
    reaches x along a residual connection."""
    rows, Cn = x2.shape
    if not on_gpu(x2):
        xf, gf, wf = x2.float(), dy2.float(), w.float()
        mean, rstd = stats[:, 0:1], stats[:, 1:2]
        xhat = (xf - mean) * rstd
        a = gf * wf
        s1 = torch.zeros(rows, 1) if rms else a.mean(1, keepdim=True)
        s2 = (a * xhat).mean(1, keepdim=True)
        dx = rstd * (a - s1 - xhat * s2)
        if dres is not None:
            dx = dx + dres.float()
        return dx.to(x2.dtype), (gf * xhat).sum(0), gf.sum(0)
    dy2 = dy2.contiguous()
    dx = torch.empty_like(x2)
    st = _lib.stream_ptr()
    if dres is not None:
        dres = dres.contiguous()
        _lib.call("nkb_norm_bwd_dx_res", dy2.data_ptr(), x2.data_ptr(), w.data_ptr(),
                  stats.data_ptr(), dx.data_ptr(), rows, Cn, int(rms), dres.data_ptr(), st)
    else:
        _lib.call("nkb_norm_bwd_dx", dy2.data_ptr(), x2.data_ptr(), w.data_ptr(), stats.data_ptr(),
                  dx.data_ptr(), rows, Cn, int(rms), st)
    acc = None
    if need_wgrad or need_bgrad:
        acc = torch.zeros(2, Cn, dtype=torch.float32, device=x2.device)
        _lib.call("nkb_colsum", dy2.data_ptr(), x2.data_ptr(), stats.data_ptr(), acc.data_ptr(),
                  rows, Cn, Cn, int(rms), st)
        _lib.count_launch()
    _lib.count_launch()
    return dx, (acc[0] if acc is not None else None), (acc[1] if acc is not None else None)


def _store_f32_grad(p, g32):
    def compute(out, accumulate):
        if out is None:
            return g32.to(p.dtype)
        if out.is_cuda and out.dtype == torch.bfloat16 and g32.is_contiguous():
            _lib.call("nkb_f32_to_bf16", g32.data_ptr(), out.data_ptr(), g32.numel(),
                      int(accumulate), _lib.stream_ptr())
            _lib.count_launch()
        else:
            out.copy_(((out.float() + g32) if accumulate else g32).to(out.dtype))
        return out
    return _deliver_grad(p, compute)


class NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps, rms):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y, stats = norm_fwd(x2, w, b, eps, rms)
        ctx.save_for_backward(x2, w, stats)
        ctx.rms = rms
        ctx.b_ref = b
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dres=None):
        x2, w, stats = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dres is not None:
            dres = dres.reshape(-1, dres.shape[-1])
        b = ctx.b_ref
        bf16_targets = all(t is None or (getattr(t, "_nkb_grad", t).dtype == torch.bfloat16)
                           for t in (w, b))
        if not on_gpu(x2) or not bf16_targets:
            dx, dw32, db32 = norm_bwd(dy2, x2, w, stats, ctx.rms, dres=dres)
            dw = _store_f32_grad(w, dw32)
            db = _store_f32_grad(b, db32) if b is not None else None
            return dx.view(dy.shape), dw, db, None, None
        # GPU: dx kernel, then one column-sum kernel that writes both parameter gradients as
        # bf16 straight into their destination (flat gradient buffer or a fresh tensor)
        dx, _, _ = norm_bwd(dy2, x2, w, stats, ctx.rms, need_wgrad=False, need_bgrad=False,
                            dres=dres)
        dy2 = dy2.contiguous()
        rows, Cn = x2.shape
        tgt_w, acc_w, ret_w = _grad_target(w)
        tgt_b, acc_b, ret_b = _grad_target(b) if b is not None else (None, False, None)
        acc, tickets = colsum_scratch(Cn, x2.device)
        _lib.call("nkb_colsum_fused", dy2.data_ptr(), x2.data_ptr(), stats.data_ptr(),
                  acc.data_ptr(), tickets.data_ptr(), tgt_w.data_ptr(), ptr(tgt_b), int(acc_w),
                  int(acc_b), rows, Cn, Cn, int(ctx.rms), _lib.stream_ptr())
        _lib.count_launch()
        _grad_done(w)
        if b is not None:
            _grad_done(b)
        return dx.view(dy.shape), ret_w, ret_b, None, None


def _grad_target(p):
    """(tensor the kernel writes, accumulate?, what autograd gets) for parameter ``p``."""
    buf = getattr(p, "_nkb_grad", None)
    if buf is None:
        out = torch.empty_like(p)
        return out, False, out
    return buf, bool(getattr(p, "_nkb_grad_has", False)), None


def _grad_done(p):
    if getattr(p, "_nkb_grad", None) is None:
        return
    p._nkb_grad_has = True
    cb = getattr(p, "_nkb_grad_ready", None)
    if cb is not None:
        cb(p)


class NormSplitFn(torch.autograd.Function):
    """``(x_alias, y) = (x, norm(x))``: the residual branch takes ``x_alias``.  Both gradients
    arrive in one backward call, so the residual-path gradient is added inside the norm
    backward kernel instead of by a separate accumulation kernel."""

    @staticmethod
    def forward(ctx, x, w, b, eps, rms):
        y = NormFn.forward(ctx, x, w, b, eps, rms)
        return x.view_as(x), y

    @staticmethod
    def backward(ctx, dres, dy):
        if dy is None:  # only the residual branch was used
            return dres, None, None, None, None
        return NormFn.backward(ctx, dy, dres)


class LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, bias: bool = True, dtype=torch.bfloat16,
                 device=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device)) if bias else None

    def forward(self, x):
        return NormFn.apply(x, self.weight, self.bias, self.eps, False)

    def split(self, x):
        """``(x, norm(x))`` for a pre-norm residual block (see ``NormSplitFn``)."""
        return NormSplitFn.apply(x, self.weight, self.bias, self.eps, False)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))

    def forward(self, x):
        return NormFn.apply(x, self.weight, None, self.eps, True)

    def split(self, x):
        """``(x, norm(x))`` for a pre-norm residual block (see ``NormSplitFn``)."""
        return NormSplitFn.apply(x, self.weight, None, self.eps, True)
