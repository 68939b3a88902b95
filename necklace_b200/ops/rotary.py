"""Rotary position embedding and SwiGLU operators (Llama-style blocks)."""
from __future__ import annotations

import torch

from .. import _lib
from ._common import on_gpu


def _rope_ref(qkv, H, base, sign, pos_offset=0):
    B, S, C3 = qkv.shape
    C = C3 // 3
    D = C // H
    half = D // 2
    pos = torch.arange(S, dtype=torch.float32, device=qkv.device) + pos_offset
    inv = base ** (-2.0 * torch.arange(half, dtype=torch.float32, device=qkv.device) / D)
    ang = pos[:, None] * inv[None, :]
    cos, sin = ang.cos()[None, :, None, :], (sign * ang.sin())[None, :, None, :]
    out = qkv.clone()
    for w in range(2):
        x = qkv[..., w * C:(w + 1) * C].float().view(B, S, H, D)
        a, b = x[..., :half], x[..., half:]
        y = torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
        out[..., w * C:(w + 1) * C] = y.view(B, S, C).to(qkv.dtype)
    return out


class LinearRopeFn(torch.autograd.Function):
    """``qkv = x @ w^T`` followed by the rotation of its q and k parts, done in place on
    the GEMM output (no extra copy); backward un-rotates the incoming gradient in place
    and feeds the projection's data- and weight-gradient GEMMs."""

    @staticmethod
    def forward(ctx, x, w, H, base, pos_offset):
        from .gemm import gemm
        x2 = x.reshape(-1, x.shape[-1])
        qkv = gemm(x2, w).view(*x.shape[:-1], w.shape[0])
        _apply(qkv, H, base, False, pos_offset)
        ctx.save_for_backward(x2, w)
        ctx.H, ctx.base, ctx.pos_offset = H, base, pos_offset
        return qkv

    @staticmethod
    def backward(ctx, dqkv):
        from .gemm import _deliver_grad, gemm
        x2, w = ctx.saved_tensors
        d = dqkv if dqkv.is_contiguous() else dqkv.contiguous()
        if not d.is_cuda:
            d = d.clone()
        d = _apply(d, ctx.H, ctx.base, True, ctx.pos_offset)
        d2 = d.reshape(-1, d.shape[-1])
        dx = gemm(d2, w, b_mn=True).view(*dqkv.shape[:-1], w.shape[1])
        dw = _deliver_grad(w, lambda out, acc: gemm(d2, x2, a_mn=True, b_mn=True, out=out,
                                                    accumulate=acc))
        return dx, dw, None, None, None


def _apply(qkv, H, base, backward, pos_offset):
    B, S, C3 = qkv.shape
    D = C3 // 3 // H
    if not on_gpu(qkv):
        qkv.copy_(_rope_ref(qkv, H, base, -1.0 if backward else 1.0, pos_offset))
        return qkv
    assert qkv.dtype == torch.bfloat16 and qkv.is_contiguous()
    _lib.call("nkb_rope", qkv.data_ptr(), B * S, S, H, D, float(base), int(backward),
              int(pos_offset), _lib.stream_ptr())
    _lib.count_launch()
    return qkv


class RopeFn(torch.autograd.Function):
    """Rotation of the q and k parts of a packed ``[B, S, 3C]`` projection, in place."""

    @staticmethod
    def forward(ctx, qkv, H, base, pos_offset):
        ctx.H, ctx.base, ctx.pos_offset = H, base, pos_offset
        ctx.mark_dirty(qkv)
        return _apply(qkv, H, base, False, pos_offset)

    @staticmethod
    def backward(ctx, d):
        d = d.contiguous()
        if not d.is_cuda:
            d = d.clone()
        return _apply(d, ctx.H, ctx.base, True, ctx.pos_offset), None, None, None


def rope(qkv, n_head, base=10000.0, pos_offset=0):
    """Rotary embedding on an already computed packed projection (used where the projection
    is a fused all-gather + GEMM)."""
    return RopeFn.apply(qkv, n_head, base, pos_offset)


def linear_rope(x, w, n_head, base=10000.0, pos_offset=0):
    """Packed QKV projection (``w`` = ``[q; k; v]`` rows, no bias) with rotary q / k."""
    return LinearRopeFn.apply(x, w, n_head, base, pos_offset)


class SwiGLUFn(torch.autograd.Function):
    """``h = silu(gu[..., :F]) * gu[..., F:]``"""

    @staticmethod
    def forward(ctx, gu):
        F_ = gu.shape[-1] // 2
        ctx.save_for_backward(gu)
        g2 = gu.reshape(-1, 2 * F_)
        if not on_gpu(gu):
            g, u = g2[:, :F_].float(), g2[:, F_:].float()
            return (torch.nn.functional.silu(g) * u).to(gu.dtype).view(*gu.shape[:-1], F_)
        h = torch.empty(g2.shape[0], F_, dtype=gu.dtype, device=gu.device)
        _lib.call("nkb_swiglu_fwd", g2.data_ptr(), h.data_ptr(), g2.shape[0], F_,
                  _lib.stream_ptr())
        _lib.count_launch()
        return h.view(*gu.shape[:-1], F_)

    @staticmethod
    def backward(ctx, dh):
        (gu,) = ctx.saved_tensors
        F_ = gu.shape[-1] // 2
        g2, d2 = gu.reshape(-1, 2 * F_), dh.reshape(-1, F_).contiguous()
        if not on_gpu(gu):
            g, u, d = g2[:, :F_].float(), g2[:, F_:].float(), d2.float()
            s = torch.sigmoid(g)
            dg = d * u * s * (1 + g * (1 - s))
            du = d * g * s
            return torch.cat([dg, du], -1).to(gu.dtype).view(gu.shape)
        dgu = torch.empty_like(g2)
        _lib.call("nkb_swiglu_bwd", g2.data_ptr(), d2.data_ptr(), dgu.data_ptr(), g2.shape[0],
                  F_, _lib.stream_ptr())
        _lib.count_launch()
        return dgu.view(gu.shape)


def swiglu(gu):
    return SwiGLUFn.apply(gu.contiguous())
