"""Tensor parallelism on the fused GEMM + collective kernels (sequence-parallel layout).

Activations between tensor-parallel regions are kept row-sharded (``[tokens/p, C]`` per
rank).  A column-parallel linear is then "all-gather rows, multiply by my weight
columns" and a row-parallel linear "multiply, reduce-scatter rows":

    ColumnParallel   fwd  Y   = AG(X) W_r^T          one kernel: ``PeerGroup.ag_gemm``
                     bwd  dX  = RS(dY W_r)           one kernel: ``PeerGroup.gemm_rs``
                          dW_r = dY^T AG(X)
    RowParallel      fwd  Y_r = RS(X W_r^T) (+b,+res) one kernel: ``PeerGroup.gemm_rs``
                     bwd  dX  = AG(dY_r) W_r         one kernel: ``PeerGroup.ag_gemm``
                          dW_r = AG(dY_r)^T X

so every collective of the reference's Megatron-style layers
(necklace/frmwrk/pytorch/mpnn/mappings.py:25-82, layers.py:239-249, :314-328) overlaps the
tensor-core work of the GEMM it belongs to, tile by tile, instead of running as a separate
blocking NCCL call.  ``group`` is a ``PeerGroup``; with one rank the plain GEMM is used.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops.gemm import _deliver_grad, colsum, gemm


class _Bufs:
    """Per-group gather buffers in the symmetric heap, keyed by shape (allocated once)."""

    def __init__(self):
        self.d = {}

    def get(self, group, rows, cols, tag, dtype=torch.bfloat16, device=None):
        key = (id(group), rows, cols, tag, dtype)
        t = self.d.get(key)
        if t is None:
            heap = getattr(group, "heap", None)
            if heap is not None:
                t = heap.alloc(rows * cols, dtype).view(rows, cols)
            else:          # torch.distributed stand-in group (CPU tests, NCCL baseline)
                t = torch.zeros(rows, cols, dtype=dtype, device=device)
            self.d[key] = t
        return t


_BUFS = _Bufs()


class AGLinearFn(torch.autograd.Function):
    """``y[M, N_r] = all_gather_rows(x_shard)[M, K] @ w_r[N_r, K]^T (+ bias)``"""

    @staticmethod
    def forward(ctx, x_shard, w, bias, group):
        p, r = group.world, group.rank
        R, K = x_shard.shape
        ctx.group = group
        if p == 1:
            y = gemm(x_shard, w, bias=bias)
            ctx.save_for_backward(x_shard, w)
            ctx.b_ref = bias
            return y
        xf = _BUFS.get(group, p * R, K, "ag_fwd", x_shard.dtype, x_shard.device)
        xf[r * R:(r + 1) * R].copy_(x_shard)
        y = group.ag_gemm(xf, w, bias=bias)
        ctx.save_for_backward(xf.clone(), w)   # gathered input, needed by the weight gradient
        ctx.b_ref = bias
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, w = ctx.saved_tensors
        group = ctx.group
        dy = dy.contiguous()
        if group.world == 1:
            dx = gemm(dy, w, b_mn=True)
        else:
            dx = group.gemm_rs(dy, w, b_mn=True)          # [M/p, K]
        dw = _deliver_grad(w, lambda out, acc: gemm(dy, x_full, a_mn=True, b_mn=True, out=out,
                                                    accumulate=acc))
        db = None
        if ctx.b_ref is not None:
            db = _deliver_grad(ctx.b_ref, lambda out, acc: colsum(dy, out, acc))
        return dx, dw, db, None


class LinearRSFn(torch.autograd.Function):
    """``y_shard[M/p, N] = reduce_scatter_rows(x[M, K_r] @ w_r[N, K_r]^T) (+ bias + residual)``"""

    @staticmethod
    def forward(ctx, x, w, bias, residual, group):
        ctx.group = group
        ctx.save_for_backward(x, w)
        ctx.b_ref, ctx.has_res = bias, residual is not None
        if group.world == 1:
            return gemm(x, w, bias=bias, res=residual)
        return group.gemm_rs(x.contiguous(), w, bias=bias, res=residual)

    @staticmethod
    def backward(ctx, dy_shard):
        x, w = ctx.saved_tensors
        group = ctx.group
        p, r = group.world, group.rank
        dy_shard = dy_shard.contiguous()
        if p == 1:
            dy_full = dy_shard
            dx = gemm(dy_full, w, b_mn=True)
        else:
            R, N = dy_shard.shape
            dyf = _BUFS.get(group, p * R, N, "ag_bwd", dy_shard.dtype, dy_shard.device)
            dyf[r * R:(r + 1) * R].copy_(dy_shard)
            dx = group.ag_gemm(dyf, w, b_mn=True)         # [M, K_r]; also fills dyf
            dy_full = dyf
        dw = _deliver_grad(w, lambda out, acc: gemm(dy_full, x, a_mn=True, b_mn=True, out=out,
                                                    accumulate=acc))
        db = None
        if ctx.b_ref is not None:
            # bias is added once after the reduction: its gradient is the column sum of the
            # local rows, summed over ranks by the data-/tensor-parallel gradient reduction
            db = _deliver_grad(ctx.b_ref, lambda out, acc: colsum(dy_shard, out, acc))
        dres = dy_shard if ctx.has_res else None
        return dx, dw, db, dres, None


def ag_linear(x_shard, w, bias, group):
    return AGLinearFn.apply(x_shard, w, bias, group)


def linear_rs(x, w, bias, residual, group):
    return LinearRSFn.apply(x, w, bias, residual, group)


class SPColumnParallelLinear(nn.Module):
    """Column-parallel linear over row-sharded input (fused all-gather -> GEMM)."""

    def __init__(self, in_features, out_features, group, bias=True, dtype=torch.bfloat16,
                 device=None, seed=1234, std=0.02):
        super().__init__()
        p, r = group.world, group.rank
        assert out_features % p == 0
        g = torch.Generator().manual_seed(seed)
        full = torch.randn(out_features, in_features, generator=g) * std
        self.group = group
        self.weight = nn.Parameter(full.chunk(p, 0)[r].contiguous().to(dtype).to(device))
        self.bias = nn.Parameter(torch.zeros(out_features // p, dtype=dtype, device=device)) \
            if bias else None
        self.weight.model_parallel, self.weight.partition_dim = True, 0
        if self.bias is not None:
            self.bias.model_parallel, self.bias.partition_dim = True, 0

    def forward(self, x_shard):
        return ag_linear(x_shard, self.weight, self.bias, self.group)


class SPRowParallelLinear(nn.Module):
    """Row-parallel linear producing row-sharded output (fused GEMM -> reduce-scatter)."""

    def __init__(self, in_features, out_features, group, bias=True, dtype=torch.bfloat16,
                 device=None, seed=4321, std=0.02):
        super().__init__()
        p, r = group.world, group.rank
        assert in_features % p == 0
        g = torch.Generator().manual_seed(seed)
        full = torch.randn(out_features, in_features, generator=g) * std
        self.group = group
        self.weight = nn.Parameter(full.chunk(p, 1)[r].contiguous().to(dtype).to(device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) \
            if bias else None
        self.weight.model_parallel, self.weight.partition_dim = True, 1

    def forward(self, x, residual=None):
        return linear_rs(x, self.weight, self.bias, residual, self.group)


# --------------------------------------------------------------- vocabulary-parallel ends
class VocabParallelEmbedFn(torch.autograd.Function):
    """Token embedding with the vocabulary rows split over the group; output row-sharded.

    Every rank looks the whole index tensor up in its slice (rows it does not own give zeros,
    as in the reference's masked lookup, necklace/frmwrk/pytorch/mpnn/layers.py:115-131); the
    reference then all-reduces the full ``[T, C]`` result, here the peer-memory reduce-scatter
    kernel leaves each rank with its ``[T/p, C]`` rows, which is what the first fused
    all-gather -> GEMM of the block wants.  Backward: all-gather the row gradients, scatter-add
    the rows this slice owns."""

    @staticmethod
    def forward(ctx, idx, wte, group):
        from ..ops.loss import embed_fwd
        p, r = group.world, group.rank
        T, S = idx.numel(), idx.shape[-1]
        Vl, Cn = wte.shape
        ctx.group, ctx.S, ctx.wte = group, S, wte
        ctx.save_for_backward(idx)
        if p == 1:
            return embed_fwd(idx, wte, None, S)
        part = _BUFS.get(group, T, Cn, "emb", wte.dtype, wte.device)
        embed_fwd(idx, wte, None, S, vocab_start=r * Vl, out=part)
        return group.reduce_scatter(part)

    @staticmethod
    def backward(ctx, dout):
        from ..ops.loss import embed_bwd
        (idx,) = ctx.saved_tensors
        group, wte = ctx.group, ctx.wte
        p, r = group.world, group.rank
        Vl, Cn = wte.shape
        dout = dout.contiguous()
        if p > 1:
            R = dout.shape[0]
            full = _BUFS.get(group, p * R, Cn, "emb", dout.dtype, dout.device)
            full[r * R:(r + 1) * R].copy_(dout)
            group.all_gather(full)
            dout = full
        buf = getattr(wte, "_nkb_grad", None)
        if buf is not None:
            if not getattr(wte, "_nkb_grad_has", False):
                buf.zero_()
            embed_bwd(idx, dout, buf, None, ctx.S, vocab_start=r * Vl)
            wte._nkb_grad_has = True
            cb = getattr(wte, "_nkb_grad_ready", None)
            if cb is not None:
                cb(wte)
            return None, None, None
        g = torch.zeros_like(wte)
        embed_bwd(idx, dout, g, None, ctx.S, vocab_start=r * Vl)
        return None, g, None


class VocabParallelLMHeadLossFn(torch.autograd.Function):
    """Mean cross-entropy of ``all_gather_rows(x) @ W_r^T`` with the vocabulary split over the
    group.  Logits exist only as this rank's ``[T, V/p]`` bf16 slice; the softmax statistics
    of the slices (max, sum of exponentials, target logit) are exchanged as a ``[p, T, 3]``
    fp32 all-gather and combined locally, then every slice turns into its own gradient in
    place.  Forward: fused all-gather -> GEMM; backward: fused GEMM -> reduce-scatter for
    dx and a plain GEMM for dW_r."""

    @staticmethod
    def forward(ctx, x_shard, w, targets, vocab, group):
        from ..ops.loss import ce_grad, ce_stats
        p, r = group.world, group.rank
        R, K = x_shard.shape
        Vl = w.shape[0]
        tg = targets.reshape(-1).contiguous()
        T = tg.numel()
        if p == 1:
            x_full = x_shard
            logits = gemm(x_shard, w)
        else:
            xf = _BUFS.get(group, p * R, K, "ag_fwd", x_shard.dtype, x_shard.device)
            xf[r * R:(r + 1) * R].copy_(x_shard)
            logits = group.ag_gemm(xf, w)
            x_full = xf.clone()
        v_lo = r * Vl
        v_local = max(0, min(Vl, vocab - v_lo))      # the last slice may hold padding rows
        st = ce_stats(logits, tg, v_local, v_lo)                      # [T, 3]
        if p > 1:
            allst = _BUFS.get(group, p * T, 4, "ce_stats", torch.float32, st.device)
            allst.view(p, T, 4)[r, :, :3].copy_(st)
            group.all_gather(allst)
            a = allst.view(p, T, 4)
            m = a[:, :, 0].max(0).values
            ssum = (a[:, :, 1] * torch.exp(a[:, :, 0] - m)).sum(0)
            tl = a[:, :, 2].sum(0)
        else:
            m, ssum, tl = st[:, 0], st[:, 1], st[:, 2]
        valid = tg >= 0
        n_valid = valid.sum().clamp(min=1).to(torch.float32)
        losses = (m + torch.log(ssum) - tl) * valid
        ce_grad(logits, tg, torch.stack([m, ssum], 1), v_local, v_lo, 1.0 / T)
        ctx.save_for_backward(x_full, w, logits, n_valid)
        ctx.group, ctx.T = group, T
        return losses.sum() / n_valid

    @staticmethod
    def backward(ctx, dloss):
        x_full, w, dlogits, n_valid = ctx.saved_tensors
        group = ctx.group
        corr = (dloss.float() * (ctx.T / n_valid)).reshape(1)
        if group.world == 1:
            dx = gemm(dlogits, w, b_mn=True, alpha_dev=corr)
        else:
            # the scalar is folded into dlogits' consumer GEMMs: gemm_rs has no device alpha,
            # so scale the (small) reduced rows instead
            dx = group.gemm_rs(dlogits, w, b_mn=True)
            dx = dx * corr.to(dx.dtype)
        dw = _deliver_grad(w, lambda out, acc: gemm(dlogits, x_full, a_mn=True, b_mn=True,
                                                    out=out, accumulate=acc, alpha_dev=corr))
        return dx, dw, None, None, None


def vocab_parallel_embed(idx, wte, group):
    return VocabParallelEmbedFn.apply(idx, wte, group)


def vocab_parallel_lm_head_loss(x_shard, w, targets, vocab, group):
    return VocabParallelLMHeadLossFn.apply(x_shard, w, targets, vocab, group)


class ReplicatedGradSync:
    """Sums, over the tensor-parallel group, the gradients of the parameters that are
    replicated on every rank of it (norm weights).  In the sequence-parallel layout each rank
    normalises only its own rows, so each rank holds only its rows' share of those gradients.
    One call per optimizer step, after the last backward: the gradients (views into the flat
    gradient buffer, or ``.grad``) are packed into one staging buffer in the symmetric heap,
    reduced by the peer-memory all-reduce kernel and unpacked, i.e. three launches however
    many norm layers there are."""

    def __init__(self, params, group):
        self.params = [p for p in params if p.requires_grad]
        self.group = group
        self.sizes = [p.numel() for p in self.params]
        n = sum(self.sizes)
        self.n = n
        self.buf = None
        if self.params and group.world > 1:
            p0 = self.params[0]
            heap = getattr(group, "heap", None)
            npad = (n + 127) // 128 * 128
            self.buf = heap.alloc(npad, p0.dtype) if heap is not None else \
                torch.zeros(npad, dtype=p0.dtype, device=p0.device)

    def _grads(self):
        out = []
        for p in self.params:
            g = getattr(p, "_nkb_grad", None)
            if g is None:
                g = p.grad
            out.append(g)
        return out

    def __call__(self):
        if self.buf is None:
            return
        grads = self._grads()
        if any(g is None for g in grads):
            return
        torch.cat([g.reshape(-1) for g in grads], out=self.buf[:self.n])
        self.group.all_reduce(self.buf)
        torch._foreach_copy_([g.reshape(-1) for g in grads], list(self.buf[:self.n].split(self.sizes)))


# ------------------------------------------ replicated-activation (Megatron) layout, fused
class ColumnLinearFn(torch.autograd.Function):
    """Column-parallel linear on a replicated input: ``y_r = x W_r^T (+ b_r)``; the input
    gradient ``sum_r dy_r W_r`` is the fused GEMM -> reduce-scatter followed by the
    peer-memory all-gather (the reference all-reduces it over NCCL after a cuBLAS GEMM,
    necklace/frmwrk/pytorch/mpnn/mappings.py:85-94)."""

    @staticmethod
    def forward(ctx, x2, w, bias, group):
        ctx.group, ctx.b_ref = group, bias
        ctx.save_for_backward(x2, w)
        return gemm(x2, w, bias=bias)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        group = ctx.group
        dy = dy.contiguous()
        M, K = x2.shape
        p, r = group.world, group.rank
        dx = None
        if ctx.needs_input_grad[0]:
            R = M // p
            full = _BUFS.get(group, M, K, "col_dx", dy.dtype, dy.device)
            group.gemm_rs(dy, w, b_mn=True, out=full[r * R:(r + 1) * R])
            group.all_gather(full)
            dx = full.clone()
        dw = _deliver_grad(w, lambda out, acc: gemm(dy, x2, a_mn=True, b_mn=True, out=out,
                                                    accumulate=acc))
        db = None
        if ctx.b_ref is not None:
            db = _deliver_grad(ctx.b_ref, lambda out, acc: colsum(dy, out, acc))
        return dx, dw, db, None


class RowLinearFn(torch.autograd.Function):
    """Row-parallel linear with a replicated output: ``y = sum_r x_r W_r^T`` as the fused
    GEMM -> reduce-scatter plus the peer-memory all-gather; backward needs no collective."""

    @staticmethod
    def forward(ctx, x2, w, group):
        ctx.group = group
        ctx.save_for_backward(x2, w)
        M, N = x2.shape[0], w.shape[0]
        p, r = group.world, group.rank
        R = M // p
        full = _BUFS.get(group, M, N, "row_y", x2.dtype, x2.device)
        group.gemm_rs(x2.contiguous(), w, out=full[r * R:(r + 1) * R])
        group.all_gather(full)
        return full.clone()

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = gemm(dy, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = _deliver_grad(w, lambda out, acc: gemm(dy, x2, a_mn=True, b_mn=True, out=out,
                                                    accumulate=acc))
        return dx, dw, None


def fused_group_of(mp_group_info, x: torch.Tensor, rows: int):
    """The ``PeerGroup`` to run the fused tensor-parallel kernels on, or None when the plain
    collective path must be taken (no peer heap, CPU tensors, not bf16, or a row count that
    does not split into 128-row blocks per rank)."""
    peer = getattr(getattr(mp_group_info, "comm", None), "peer", None)
    if peer is None or not x.is_cuda or x.dtype != torch.bfloat16:
        return None
    if rows % (128 * peer.world):
        return None
    return peer
