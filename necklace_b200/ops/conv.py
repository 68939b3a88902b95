"""Convolution, batch norm (+ residual + ReLU) and pooling on channels-last bf16 tensors.

Tensors are ``[N, H, W, C]`` (NHWC) everywhere, so a 1x1 convolution is a GEMM on the
activation matrix as it is and every other convolution is a GEMM on a gathered ``col``
matrix; all GEMMs run on the tcgen05 kernel (``ops.gemm``).  Weights are stored
``[C_out, KH*KW*C_in]`` with the input channel innermost, which is what that GEMM wants as
its K-major B operand.  CPU tensors take PyTorch reference paths (``F.conv2d`` and friends
on permuted views), which the CPU test-suite and the GPU numerics tests compare against.

These operators replace the cuDNN convolutions / batch norm / pooling the reference's CNN
examples use through torch (examples/dp/mnist/pytorch/main.py) for the ResNet-50
data-parallel configuration.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _lib
from ._common import on_gpu, ptr, scratch, scratch_zero
from .gemm import _deliver_grad, gemm


def _out_hw(H, W, KH, KW, stride, pad):
    return (H + 2 * pad - KH) // stride + 1, (W + 2 * pad - KW) // stride + 1


def _kpad(KH, KW, C):
    return (KH * KW * C + 7) // 8 * 8


def im2col(x: torch.Tensor, KH: int, KW: int, stride: int, pad: int, out=None) -> torch.Tensor:
    """``x`` [N,H,W,C] -> col [N*Ho*Wo, Kpad] with K index ``(kh*KW + kw)*C + c``."""
    N, H, W, C = x.shape
    Ho, Wo = _out_hw(H, W, KH, KW, stride, pad)
    Kp = _kpad(KH, KW, C)
    M = N * Ho * Wo
    if not on_gpu(x):
        cols = F.unfold(x.permute(0, 3, 1, 2).float(), (KH, KW), padding=pad, stride=stride)
        # unfold: [N, C*KH*KW, L] with index c*KH*KW + tap  ->  [N*L, tap*C + c]
        cols = cols.view(N, C, KH * KW, Ho * Wo).permute(0, 3, 2, 1).reshape(M, KH * KW * C)
        res = torch.zeros(M, Kp, dtype=x.dtype)
        res[:, :KH * KW * C] = cols.to(x.dtype)
        return res
    assert x.dtype == torch.bfloat16 and x.is_contiguous()
    if out is None:
        out = torch.empty(M, Kp, dtype=x.dtype, device=x.device)
    _lib.call("nkb_im2col_nhwc", x.data_ptr(), out.data_ptr(), N, H, W, C, KH, KW, stride, pad, Kp,
              _lib.stream_ptr())
    _lib.count_launch()
    return out


def col2im(dcol: torch.Tensor, shape, KH: int, KW: int, stride: int, pad: int) -> torch.Tensor:
    """Adjoint of ``im2col``: dcol [N*Ho*Wo, Kpad] -> dx [N,H,W,C]."""
    N, H, W, C = shape
    Ho, Wo = _out_hw(H, W, KH, KW, stride, pad)
    Kp = _kpad(KH, KW, C)
    if not on_gpu(dcol):
        d = dcol[:, :KH * KW * C].float().view(N, Ho * Wo, KH * KW, C).permute(0, 3, 2, 1)
        d = d.reshape(N, C * KH * KW, Ho * Wo)
        dx = F.fold(d, (H, W), (KH, KW), padding=pad, stride=stride)
        return dx.permute(0, 2, 3, 1).contiguous().to(dcol.dtype)
    dx = torch.empty(N, H, W, C, dtype=dcol.dtype, device=dcol.device)
    _lib.call("nkb_col2im_nhwc", dcol.data_ptr(), dx.data_ptr(), N, H, W, C, KH, KW, stride, pad,
              Kp, _lib.stream_ptr())
    _lib.count_launch()
    return dx


class Conv2dFn(torch.autograd.Function):
    """``y[N,Ho,Wo,Cout] = conv(x[N,H,W,Cin], w[Cout, KH*KW*Cin (padded to 8)])``, no bias."""

    @staticmethod
    def forward(ctx, x, w, KH, KW, stride, pad):
        N, H, W, C = x.shape
        Ho, Wo = _out_hw(H, W, KH, KW, stride, pad)
        ctx.geom = (KH, KW, stride, pad)
        ctx.xshape = tuple(x.shape)
        direct = KH == 1 and KW == 1 and stride == 1 and pad == 0 and C % 8 == 0
        ctx.direct = direct
        a = x.reshape(-1, C) if direct else im2col(x, KH, KW, stride, pad)
        y = gemm(a, w)
        # the gathered matrix is kept for the weight gradient unless it would be very large
        # (then it is rebuilt in backward): KH*KW times the input, which 180 GB of HBM affords
        keep = (not direct) and a.numel() * a.element_size() <= Conv2dFn.KEEP_COL_BYTES
        ctx.keep_col = keep
        if keep:
            ctx.save_for_backward(x, w, a)
        else:
            ctx.save_for_backward(x, w)
        return y.view(N, Ho, Wo, w.shape[0])

    KEEP_COL_BYTES = 2 << 30

    @staticmethod
    def backward(ctx, dy):
        if ctx.keep_col:
            x, w, col = ctx.saved_tensors
        else:
            (x, w), col = ctx.saved_tensors, None
        KH, KW, stride, pad = ctx.geom
        N, H, W, C = ctx.xshape
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            d = gemm(dy2, w, b_mn=True)                       # [M, Kpad]
            dx = d.view(N, H, W, C) if ctx.direct else col2im(d, ctx.xshape, KH, KW, stride, pad)
        a = x.reshape(-1, C) if ctx.direct else \
            (col if col is not None else im2col(x, KH, KW, stride, pad))
        dw = _deliver_grad(w, lambda out, acc: gemm(dy2, a, a_mn=True, b_mn=True, out=out,
                                                    accumulate=acc))
        return dx, dw, None, None, None, None


def conv2d(x, w, KH, KW, stride=1, pad=0):
    return Conv2dFn.apply(x, w, KH, KW, stride, pad)


class Conv2d(nn.Module):
    """Bias-free convolution on NHWC bf16 activations."""

    def __init__(self, cin, cout, k=1, stride=1, pad=0, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cin, self.cout, self.k, self.stride, self.pad = cin, cout, k, stride, pad
        w4 = torch.empty(cout, cin, k, k)
        nn.init.kaiming_normal_(w4, mode="fan_out", nonlinearity="relu")
        w = torch.zeros(cout, _kpad(k, k, cin))
        w[:, :k * k * cin] = w4.permute(0, 2, 3, 1).reshape(cout, -1)   # (kh, kw, c) order
        self.weight = nn.Parameter(w.to(dtype).to(device) if device is not None else w.to(dtype))

    def weight_oihw(self) -> torch.Tensor:
        """The weight in torch's [Cout, Cin, KH, KW] layout (for comparisons / export)."""
        k, cin = self.k, self.cin
        return self.weight[:, :k * k * cin].view(self.cout, k, k, cin).permute(0, 3, 1, 2)

    def forward(self, x):
        return conv2d(x, self.weight, self.k, self.k, self.stride, self.pad)


# ------------------------------------------------------------------------ batch norm
def _bn_acc(C, device):
    return scratch_zero("bn_acc", 2 * 8192, torch.float32, device)


class BatchNormFn(torch.autograd.Function):
    """Training-mode batch norm over the rows of ``x [.., C]``, optionally followed by a
    residual add and ReLU, in one pass over the data after the statistics pass."""

    @staticmethod
    def forward(ctx, x, gamma, beta, res, run_mean, run_var, eps, momentum, relu):
        C = x.shape[-1]
        x2 = x.reshape(-1, C)
        M = x2.shape[0]
        r2 = res.reshape(-1, C) if res is not None else None
        if not on_gpu(x):
            xf = x2.float()
            mean = xf.mean(0)
            var = xf.var(0, unbiased=False)
            rstd = torch.rsqrt(var + eps)
            y = (xf - mean) * rstd * gamma.float() + beta.float()
            if r2 is not None:
                y = y + r2.float()
            if relu:
                y = torch.relu(y)
            if run_mean is not None:
                run_mean.mul_(1 - momentum).add_(momentum * mean)
                run_var.mul_(1 - momentum).add_(momentum * var * (M / max(M - 1, 1)))
            stats = torch.stack([mean, rstd])
            y = y.to(x.dtype)
        else:
            assert x.dtype == torch.bfloat16 and x2.is_contiguous() and C % 8 == 0 and C <= 8192
            y = torch.empty_like(x2)
            stats = torch.empty(2, C, dtype=torch.float32, device=x.device)
            _lib.call("nkb_bn_fwd", x2.data_ptr(), gamma.data_ptr(), beta.data_ptr(), ptr(r2),
                      y.data_ptr(), stats.data_ptr(), _bn_acc(C, x.device).data_ptr(),
                      ptr(run_mean), ptr(run_var), M, C, float(eps), float(momentum), int(relu),
                      _lib.stream_ptr())
            _lib.count_launch(3)
        ctx.save_for_backward(x2, y if relu else None, stats, gamma)
        ctx.refs = (gamma, beta)
        ctx.relu, ctx.has_res, ctx.shape = relu, res is not None, x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, y, stats, gamma = ctx.saved_tensors
        g_ref, b_ref = ctx.refs
        M, C = x2.shape
        dy2 = dy.reshape(-1, C)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        relu, has_res = ctx.relu, ctx.has_res
        if not on_gpu(x2):
            d = dy2.float()
            if relu:
                d = d * (y.float() > 0)
            mean, rstd = stats[0], stats[1]
            xhat = (x2.float() - mean) * rstd
            s0, s1 = d.sum(0), (d * xhat).sum(0)
            dx = gamma.float() * rstd * (d - s0 / M - xhat * s1 / M)
            dg = _deliver_grad(g_ref, lambda out, acc: _acc_into(out, s1, acc, g_ref))
            db = _deliver_grad(b_ref, lambda out, acc: _acc_into(out, s0, acc, b_ref))
            dres = d.to(dy.dtype).view(ctx.shape) if has_res else None
            return (dx.to(dy.dtype).view(ctx.shape), dg, db, dres, None, None, None, None, None)
        dx = torch.empty_like(x2)
        dres = torch.empty_like(x2) if (has_res and relu) else None
        outs = {}

        def target(p):
            buf = getattr(p, "_nkb_grad", None)
            if buf is None:
                return torch.empty_like(p), False, False
            return buf, bool(getattr(p, "_nkb_grad_has", False)), True

        gbuf, gacc, gdirect = target(g_ref)
        bbuf, bacc, bdirect = target(b_ref)
        _lib.call("nkb_bn_bwd", dy2.data_ptr(), x2.data_ptr(), ptr(y), stats.data_ptr(),
                  gamma.data_ptr(), dx.data_ptr(), ptr(dres), gbuf.data_ptr(), bbuf.data_ptr(),
                  int(gacc), int(bacc), _bn_acc(C, x2.device).data_ptr(), M, C, int(relu),
                  _lib.stream_ptr())
        _lib.count_launch(3)
        for p, direct in ((g_ref, gdirect), (b_ref, bdirect)):
            if direct:
                p._nkb_grad_has = True
                cb = getattr(p, "_nkb_grad_ready", None)
                if cb is not None:
                    cb(p)
        if has_res and dres is None:
            dres = dy2                      # no ReLU in front: the residual gets dy itself
        return (dx.view(ctx.shape), None if gdirect else gbuf, None if bdirect else bbuf,
                dres.view(ctx.shape) if has_res else None, None, None, None, None, None)


def _acc_into(out, val, acc, like):
    if out is None:
        return val.to(like.dtype)
    out.copy_(((out.float() + val) if acc else val).to(out.dtype))
    return out


class BatchNorm2d(nn.Module):
    """Batch norm over NHWC activations with optional fused residual add and ReLU:
    ``y = relu(bn(x) + residual)``.  Evaluation mode uses the running statistics."""

    def __init__(self, C, relu=False, eps=1e-5, momentum=0.1, dtype=torch.bfloat16, device=None,
                 zero_init=False):
        super().__init__()
        self.C, self.relu, self.eps, self.momentum = C, relu, eps, momentum
        self.weight = nn.Parameter(torch.zeros(C, dtype=dtype, device=device) if zero_init
                                   else torch.ones(C, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(C, dtype=dtype, device=device))
        self.register_buffer("running_mean", torch.zeros(C, dtype=torch.float32, device=device))
        self.register_buffer("running_var", torch.ones(C, dtype=torch.float32, device=device))

    def forward(self, x, residual=None):
        if self.training:
            return BatchNormFn.apply(x, self.weight, self.bias, residual, self.running_mean,
                                     self.running_var, self.eps, self.momentum, self.relu)
        stats = torch.stack([self.running_mean, torch.rsqrt(self.running_var + self.eps)])
        C = self.C
        x2 = x.reshape(-1, C)
        if not on_gpu(x):
            y = (x2.float() - stats[0]) * stats[1] * self.weight.float() + self.bias.float()
            if residual is not None:
                y = y + residual.reshape(-1, C).float()
            return (torch.relu(y) if self.relu else y).to(x.dtype).view(x.shape)
        y = torch.empty_like(x2)
        r2 = residual.reshape(-1, C) if residual is not None else None
        _lib.call("nkb_bn_apply", x2.data_ptr(), stats.contiguous().data_ptr(),
                  self.weight.data_ptr(), self.bias.data_ptr(), ptr(r2), y.data_ptr(),
                  x2.shape[0], C, int(self.relu), _lib.stream_ptr())
        _lib.count_launch()
        return y.view(x.shape)


# ---------------------------------------------------------------------------- pooling
class MaxPool3x3s2Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        N, H, W, C = x.shape
        Ho, Wo = _out_hw(H, W, 3, 3, 2, 1)
        ctx.shape = tuple(x.shape)
        if not on_gpu(x):
            y, idx = F.max_pool2d(x.permute(0, 3, 1, 2).float(), 3, 2, 1, return_indices=True)
            ctx.save_for_backward(idx)
            return y.permute(0, 2, 3, 1).contiguous().to(x.dtype)
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and C % 8 == 0
        y = torch.empty(N, Ho, Wo, C, dtype=x.dtype, device=x.device)
        idx = torch.empty(N, Ho, Wo, C, dtype=torch.uint8, device=x.device)
        _lib.call("nkb_maxpool3x3s2_fwd", x.data_ptr(), y.data_ptr(), idx.data_ptr(), N, H, W, C,
                  _lib.stream_ptr())
        _lib.count_launch()
        ctx.save_for_backward(idx)
        return y

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        N, H, W, C = ctx.shape
        if not on_gpu(dy):
            # overlapping windows: an input element can win several of them, so add up
            d = torch.zeros(N, C, H * W)
            d.scatter_add_(2, idx.reshape(N, C, -1), dy.permute(0, 3, 1, 2).float().reshape(N, C, -1))
            return d.view(N, C, H, W).permute(0, 2, 3, 1).contiguous().to(dy.dtype)
        dy = dy.contiguous()
        dx = torch.empty(N, H, W, C, dtype=dy.dtype, device=dy.device)
        _lib.call("nkb_maxpool3x3s2_bwd", dy.data_ptr(), idx.data_ptr(), dx.data_ptr(), N, H, W, C,
                  _lib.stream_ptr())
        _lib.count_launch()
        return dx


class AvgPoolFn(torch.autograd.Function):
    """Global average over H x W: [N,H,W,C] -> [N,C]."""

    @staticmethod
    def forward(ctx, x):
        N, H, W, C = x.shape
        ctx.shape = tuple(x.shape)
        if not on_gpu(x):
            return x.float().mean((1, 2)).to(x.dtype)
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and C % 8 == 0
        y = torch.empty(N, C, dtype=x.dtype, device=x.device)
        _lib.call("nkb_avgpool_fwd", x.data_ptr(), y.data_ptr(), N, H * W, C, _lib.stream_ptr())
        _lib.count_launch()
        return y

    @staticmethod
    def backward(ctx, dy):
        N, H, W, C = ctx.shape
        if not on_gpu(dy):
            return (dy.float()[:, None, None, :] / (H * W)).expand(N, H, W, C).to(dy.dtype) \
                .contiguous()
        dy = dy.contiguous()
        dx = torch.empty(N, H, W, C, dtype=dy.dtype, device=dy.device)
        _lib.call("nkb_avgpool_bwd", dy.data_ptr(), dx.data_ptr(), N, H * W, C, _lib.stream_ptr())
        _lib.count_launch()
        return dx


def max_pool_3x3_s2(x):
    return MaxPool3x3s2Fn.apply(x)


def global_avg_pool(x):
    return AvgPoolFn.apply(x)
