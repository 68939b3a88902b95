"""bf16 GEMM on tcgen05/TMEM and the linear-layer autograd functions built on it.

``gemm`` computes ``C[M,N] = epi(alpha * A[M,K] @ B[N,K]^T + bias) + res`` with either
operand allowed to be stored transposed (``a_mn`` / ``b_mn``), which is how forward,
data-gradient and weight-gradient of a linear layer all map to the same kernel
without transpose copies.  CPU tensors take a PyTorch fp32 reference path (used
by the CPU test-suite); CUDA tensors always take the native kernel.

Replaces the ``F.linear`` (cuBLAS) calls in the reference's tensor-parallel layers
(necklace/frmwrk/pytorch/mpnn/layers.py:239-249, :314-328).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _lib
from ._common import scratch_zero, on_gpu, ptr, status_word, scratch

EPI_NONE, EPI_GELU_FWD, EPI_GELU_BWD, EPI_RELU = 0, 1, 2, 3


def _gelu_tanh_grad(z: torch.Tensor) -> torch.Tensor:
    k0, k1 = 0.7978845608028654, 0.044715
    u = k0 * (z + k1 * z ** 3)
    t = torch.tanh(u)
    return 0.5 * (1 + t) + 0.5 * z * (1 - t * t) * k0 * (1 + 3 * k1 * z * z)


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
         accumulate: bool = False, alpha: float = 1.0, bias: torch.Tensor | None = None,
         res: torch.Tensor | None = None, epi: int = EPI_NONE, aux: torch.Tensor | None = None,
         ready_flags: torch.Tensor | None = None, rows_per_flag: int = 0, ready_target: int = 0,
         max_ctas: int = 0, bn: int = 0,
         alpha_dev: torch.Tensor | None = None) -> torch.Tensor:
    """``a`` is stored ``[M,K]`` (or ``[K,M]`` when ``a_mn``); ``b`` is stored ``[N,K]``
    (or ``[K,N]`` when ``b_mn``).  Both must be 2-D with unit inner stride."""
    assert a.dim() == 2 and b.dim() == 2
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
        assert not accumulate
    assert out.shape == (M, N) and out.stride(1) == 1

    if not on_gpu(a, b, out):
        A = a.float().t() if a_mn else a.float()
        B = b.float().t() if b_mn else b.float()
        y = alpha * (A @ B.t())
        if alpha_dev is not None:
            y = y * alpha_dev.float()
        if bias is not None:
            y = y + bias.float()
        if epi == EPI_GELU_FWD:
            aux.copy_(y.to(aux.dtype))
            y = F.gelu(y, approximate="tanh")
        elif epi == EPI_GELU_BWD:
            y = y * _gelu_tanh_grad(aux.float())
        elif epi == EPI_RELU:
            y = torch.relu(y)
        if res is not None:
            y = y + res.float()
        if accumulate:
            y = y + out.float()
        out.copy_(y.to(out.dtype))
        return out

    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(1) == 1 and b.stride(1) == 1
    assert out.dtype in (torch.bfloat16, torch.float32)
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.is_contiguous() and bias.numel() == N
    if res is not None:
        assert res.dtype == torch.bfloat16 and res.shape == (M, N) and res.stride(1) == 1
    if epi in (EPI_GELU_FWD, EPI_GELU_BWD):
        assert aux is not None and aux.dtype == torch.bfloat16 and aux.shape == (M, N)
        assert aux.stride(1) == 1
    # TMA: 16-byte aligned base and row pitch; repack the rare operand that is not
    if a.stride(0) % 8 or a.data_ptr() % 16:
        a = _repack(a)
    if b.stride(0) % 8 or b.data_ptr() % 16:
        b = _repack(b)
    _ensure_workspace(a.device)
    _lib.call("nkb_gemm_bf16", a.data_ptr(), a.stride(0), int(a_mn), b.data_ptr(), b.stride(0),
              int(b_mn), out.data_ptr(), out.stride(0), int(out.dtype == torch.float32),
              int(accumulate), M, N, K, float(alpha), ptr(bias), ptr(res),
              res.stride(0) if res is not None else 0, int(epi), ptr(aux),
              aux.stride(0) if aux is not None else 0, status_word(a.device).data_ptr(),
              ptr(ready_flags), int(rows_per_flag), int(ready_target), int(max_ctas), int(bn),
              ptr(alpha_dev), _lib.stream_ptr())
    _lib.count_launch()
    return out


_WORKSPACE: dict = {}
SPLITK_WORKSPACE_FLOATS = 32 * 1024 * 1024  # 128 MB: 8 slices of a 1024 x 4096 fp32 tile set


def _ensure_workspace(device) -> None:
    """Hand the library its split-K workspace (the library itself never allocates).  One
    buffer per device, owned here for the life of the process; weight-gradient GEMMs with
    few output tiles and a long K use it to spread their K range over all SMs."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx in _WORKSPACE:
        return
    ws = torch.empty(SPLITK_WORKSPACE_FLOATS, dtype=torch.float32, device=device)
    _WORKSPACE[idx] = ws
    lib = _lib.load()
    lib.nkb_gemm_set_workspace.argtypes = [_lib.vp, _lib.i64]
    lib.nkb_gemm_set_workspace.restype = None
    lib.nkb_gemm_set_workspace(ws.data_ptr(), ws.numel())


def set_splitk(enabled: bool) -> None:
    lib = _lib.load()
    lib.nkb_gemm_set_splitk.argtypes = [_lib.i32]
    lib.nkb_gemm_set_splitk.restype = None
    lib.nkb_gemm_set_splitk(int(enabled))


def _repack(t: torch.Tensor) -> torch.Tensor:
    """Copy into a buffer whose row pitch is a multiple of 8 elements (16 bytes)."""
    rows, cols = t.shape
    ld = (cols + 7) // 8 * 8
    buf = torch.zeros(rows, ld, dtype=t.dtype, device=t.device)
    buf[:, :cols].copy_(t)
    return buf[:, :cols]


def colsum(dy: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False
           ) -> torch.Tensor:
    """Bias gradient: sum of ``dy[rows, C]`` over rows, bf16 out."""
    rows, Cn = dy.shape
    if out is None:
        out = torch.empty(Cn, dtype=dy.dtype, device=dy.device)
        accumulate = False
    if not on_gpu(dy):
        s = dy.float().sum(0)
        out.copy_(((out.float() + s) if accumulate else s).to(out.dtype))
        return out
    assert dy.dtype == torch.bfloat16 and dy.stride(1) == 1
    acc, tickets = colsum_scratch(Cn, dy.device)
    _lib.call("nkb_colsum_fused", dy.data_ptr(), None, None, acc.data_ptr(), tickets.data_ptr(),
              None, out.data_ptr(), 0, int(accumulate), rows, Cn, dy.stride(0), 0,
              _lib.stream_ptr())
    _lib.count_launch()
    return out


def colsum_scratch(Cn: int, device):
    """fp32 accumulator [2][C] and ticket counters of the fused column-sum kernel; shared by
    all calls on the device's compute stream (the kernel leaves both at zero)."""
    acc = scratch_zero("colsum_acc", 2 * 65536, torch.float32, device)
    tickets = scratch_zero("colsum_tickets", 256, torch.int32, device)
    assert Cn <= 65536
    return acc, tickets


# ---------------------------------------------------------------- autograd
def _deliver_grad(p: torch.Tensor, compute):
    """Weight/bias gradient delivery.

    When the parameter carries ``_nkb_grad`` (a view into a flat gradient buffer,
    set by the flat-parameter store) the gradient kernel writes or accumulates
    straight into it and autograd gets ``None``; otherwise the fresh gradient is
    returned for autograd to accumulate.  ``_nkb_grad_ready`` (if set) is called
    once the kernel is enqueued so data-parallel buckets can start reducing while
    backward continues.
    """
    buf = getattr(p, "_nkb_grad", None)
    if buf is None:
        return compute(None, False)
    compute(buf, bool(getattr(p, "_nkb_grad_has", False)))
    p._nkb_grad_has = True
    cb = getattr(p, "_nkb_grad_ready", None)
    if cb is not None:
        cb(p)
    return None


class LinearFn(torch.autograd.Function):
    """``y = x @ w^T + b (+ residual)`` with ``w`` stored ``[out, in]``."""

    @staticmethod
    def forward(ctx, x, w, b, residual):
        x2 = x.reshape(-1, x.shape[-1])
        r2 = residual.reshape(-1, w.shape[0]) if residual is not None else None
        y = gemm(x2, w, bias=b, res=r2)
        ctx.save_for_backward(x2, w)
        ctx.has_b = b is not None
        ctx.has_r = residual is not None
        ctx.b_ref = b
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).view(*dy.shape[:-1], w.shape[1])
        if ctx.needs_input_grad[1]:
            dw = _deliver_grad(w, lambda out, acc: gemm(dy2, x2, a_mn=True, b_mn=True, out=out,
                                                        accumulate=acc))
        if ctx.has_b and ctx.needs_input_grad[2]:
            db = _deliver_grad(ctx.b_ref, lambda out, acc: colsum(dy2, out, acc))
        dres = dy if ctx.has_r and ctx.needs_input_grad[3] else None
        return dx, dw, db, dres


class MLPFn(torch.autograd.Function):
    """``y = act(x W1^T + b1) W2^T + b2 (+ residual)``, act = tanh-GELU or ReLU.

    The activation runs in the epilogue of the first GEMM (which also saves the
    pre-activation); its derivative runs in the epilogue of the data-gradient GEMM
    of the second layer, so no separate activation kernels exist in either direction.
    """

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual, act):
        x2 = x.reshape(-1, x.shape[-1])
        r2 = residual.reshape(-1, w2.shape[0]) if residual is not None else None
        if act == "gelu":
            z = torch.empty(x2.shape[0], w1.shape[0], dtype=x2.dtype, device=x2.device)
            h = gemm(x2, w1, bias=b1, epi=EPI_GELU_FWD, aux=z)
        else:
            z = None
            h = gemm(x2, w1, bias=b1, epi=EPI_RELU)
        y = gemm(h, w2, bias=b2, res=r2)
        ctx.save_for_backward(x2, w1, w2, h, z)
        ctx.act = act
        ctx.refs = (b1, b2)
        ctx.has_r = residual is not None
        return y.view(*x.shape[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w1, w2, h, z = ctx.saved_tensors
        b1, b2 = ctx.refs
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if ctx.act == "gelu":
            dz = gemm(dy2, w2, b_mn=True, epi=EPI_GELU_BWD, aux=z)
        else:
            dz = gemm(dy2, w2, b_mn=True)
            dz = dz * (h > 0).to(dz.dtype)
        dw2 = _deliver_grad(w2, lambda out, acc: gemm(dy2, h, a_mn=True, b_mn=True, out=out,
                                                      accumulate=acc))
        db2 = None
        if b2 is not None:
            db2 = _deliver_grad(b2, lambda out, acc: colsum(dy2, out, acc))
        dx = gemm(dz, w1, b_mn=True).view(*dy.shape[:-1], w1.shape[1]) \
            if ctx.needs_input_grad[0] else None
        dw1 = _deliver_grad(w1, lambda out, acc: gemm(dz, x2, a_mn=True, b_mn=True, out=out,
                                                      accumulate=acc))
        db1 = None
        if b1 is not None:
            db1 = _deliver_grad(b1, lambda out, acc: colsum(dz, out, acc))
        dres = dy if ctx.has_r else None
        return dx, dw1, db1, dw2, db2, dres, None


def linear(x, w, b=None, residual=None):
    return LinearFn.apply(x, w, b, residual)


def mlp(x, w1, b1, w2, b2, residual=None, act="gelu"):
    return MLPFn.apply(x, w1, b1, w2, b2, residual, act)


class Linear(nn.Module):
    """Drop-in ``nn.Linear`` whose matmuls run on the tcgen05 GEMM."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 dtype=torch.bfloat16, device=None, init_std: float | None = None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype,
                                               device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) \
            if bias else None
        if init_std is None:
            nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)
        else:
            nn.init.normal_(self.weight, std=init_std)

    def forward(self, x, residual=None):
        return linear(x, self.weight, self.bias, residual)
