"""Multi-head attention (causal or full) on packed QKV, forward and backward.

``attention_qkv(qkv, n_head)`` takes the fused projection output ``[B, S, 3*C]`` and
reads Q, K and V in place through strides (no split / transpose copies); the
backward writes dQ, dK, dV straight into one ``[B, S, 3*C]`` buffer that feeds the
projection's gradient GEMMs.  The reference has no attention layer; this operator
exists for the transformer configurations the benchmarks name.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .. import _lib
from ._common import on_gpu, status_word


def set_exp_mode(mode: int) -> None:
    """Forward exponentials: 0 = fp32 (default), 1 = packed half (two per MUFU op),
    2 = packed bf16 (one-tile kernel only)."""
    lib = _lib.load()
    lib.nkb_attn_set_exp_mode.argtypes = [_lib.i32]
    lib.nkb_attn_set_exp_mode.restype = None
    lib.nkb_attn_set_exp_mode(int(mode))


def set_fwd_impl(impl: int) -> None:
    """Forward kernel: 1 = ping-pong (two query tiles per CTA, P through TMEM; default),
    0 = one query tile per CTA."""
    lib = _lib.load()
    lib.nkb_attn_set_fwd_impl.argtypes = [_lib.i32]
    lib.nkb_attn_set_fwd_impl.restype = None
    lib.nkb_attn_set_fwd_impl(int(impl))


def set_bwd_impl(impl: int) -> None:
    """Backward kernel for head dim 64: 1 = warp-specialised (default), 0 = serial."""
    lib = _lib.load()
    lib.nkb_attn_set_bwd_impl.argtypes = [_lib.i32]
    lib.nkb_attn_set_bwd_impl.restype = None
    lib.nkb_attn_set_bwd_impl(int(impl))


def _ref_attention(q, k, v, causal, scale):
    # q,k,v: [B,H,S,D] fp32
    s = (q @ k.transpose(-1, -2)) * scale
    if causal:
        S = q.shape[-2]
        mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, -1)
    return p @ v


def _split(qkv, H):
    B, S, C3 = qkv.shape
    C = C3 // 3
    D = C // H
    q, k, v = (qkv[..., i * C:(i + 1) * C].view(B, S, H, D).permute(0, 2, 1, 3) for i in range(3))
    return q, k, v, B, S, C, D


def attn_fwd(qkv: torch.Tensor, H: int, causal: bool = True):
    """Returns (out [B,S,C], lse [B,H,S] fp32)."""
    q, k, v, B, S, C, D = _split(qkv, H)
    scale = 1.0 / math.sqrt(D)
    if not on_gpu(qkv):
        qf, kf, vf = q.float(), k.float(), v.float()
        s = (qf @ kf.transpose(-1, -2)) * scale
        if causal:
            s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf"))
        lse = torch.logsumexp(s, -1)
        o = torch.softmax(s, -1) @ vf
        return o.permute(0, 2, 1, 3).reshape(B, S, C).to(qkv.dtype), lse
    assert qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and D in (64, 128)
    out = torch.empty(B, S, C, dtype=qkv.dtype, device=qkv.device)
    lse = torch.empty(B, H, S, dtype=torch.float32, device=qkv.device)
    _lib.call("nkb_attn_fwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
              lse.data_ptr(), B, H, S, D, S * 3 * C, D, 3 * C, S * C, D, C, float(scale),
              int(causal), status_word(qkv.device).data_ptr(), _lib.stream_ptr())
    _lib.count_launch()
    return out, lse


def attn_bwd(qkv, out, lse, dout, H: int, causal: bool = True):
    """Returns dqkv [B,S,3C]."""
    q, k, v, B, S, C, D = _split(qkv, H)
    scale = 1.0 / math.sqrt(D)
    if not on_gpu(qkv):
        qf, kf, vf = q.float(), k.float(), v.float()
        do = dout.view(B, S, H, D).permute(0, 2, 1, 3).float()
        s = (qf @ kf.transpose(-1, -2)) * scale
        if causal:
            s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf"))
        p = torch.exp(s - lse[..., None])
        dv = p.transpose(-1, -2) @ do
        dp = do @ vf.transpose(-1, -2)
        delta = (do * (p @ vf)).sum(-1, keepdim=True)
        ds = p * (dp - delta) * scale
        dq = ds @ kf
        dk = ds.transpose(-1, -2) @ qf
        dqkv = torch.empty_like(qkv)
        for i, g in enumerate((dq, dk, dv)):
            dqkv[..., i * C:(i + 1) * C] = g.permute(0, 2, 1, 3).reshape(B, S, C).to(qkv.dtype)
        return dqkv
    dout = dout.contiguous()
    dqkv = torch.empty_like(qkv)
    dq, dk, dv, *_ = _split(dqkv, H)
    delta = torch.empty(B, H, S, dtype=torch.float32, device=qkv.device)
    dq_acc = torch.empty(B, H, S, D, dtype=torch.float32, device=qkv.device)  # cleared by the delta kernel
    _lib.call("nkb_attn_bwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
              dout.data_ptr(), lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
              delta.data_ptr(), dq_acc.data_ptr(), B, H, S, D, S * 3 * C, D, 3 * C, S * C, D, C,
              float(scale), int(causal), status_word(qkv.device).data_ptr(), _lib.stream_ptr())
    _lib.count_launch(3)
    return dqkv


class AttentionQKVFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, H, causal):
        out, lse = attn_fwd(qkv, H, causal)
        ctx.save_for_backward(qkv, out, lse)
        ctx.H, ctx.causal = H, causal
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        return attn_bwd(qkv, out, lse, dout, ctx.H, ctx.causal), None, None


def attention_qkv(qkv: torch.Tensor, n_head: int, causal: bool = True) -> torch.Tensor:
    return AttentionQKVFn.apply(qkv, n_head, causal)
