"""2-bit threshold gradient codec (with error feedback).

Arithmetic follows the reference's numba kernels (necklace/cuda/quantize.py:16-91):
``a >= thr -> code 1 -> +thr``, ``a <= -thr -> code 2 -> -thr``, else ``0``; sixteen
2-bit codes per ``uint32``, element ``i`` at bits ``[2i, 2i+2)``.  ``*_flat`` pack 16
consecutive elements of a flat vector (the layout the fused data-parallel
all-reduce uses); ``matrix_*`` pack 16 *rows* of one column, which is the layout
of the reference wrappers ``cu_fn_matrix_quantize_e`` / ``cu_fn_matrix_dequantize_e``
(quantize.py:96-134) but without their 512x512 size limit.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import _lib
from ._common import on_gpu

CMP_RATIO = 16


def _codes_cpu(a: torch.Tensor, thr: float):
    pos, neg = a >= thr, a <= -thr
    code = pos.to(torch.int64) + 2 * (neg & ~pos).to(torch.int64)
    resid = torch.where(pos, a - thr, torch.where(neg, a + thr, a))
    return code, resid


def quantize_flat(g: torch.Tensor, residual: torch.Tensor, thr: float,
                  codes: torch.Tensor | None = None) -> torch.Tensor:
    """``residual`` (fp32, same numel) is read, added to ``g`` and overwritten."""
    n = g.numel()
    nw = (n + 15) // 16
    if codes is None:
        codes = torch.empty(nw, dtype=torch.int32, device=g.device)
    if not on_gpu(g):
        a = g.reshape(-1).float() + residual.reshape(-1)
        code, res = _codes_cpu(a, thr)
        residual.reshape(-1).copy_(res)
        pad = torch.zeros(nw * 16, dtype=torch.int64)
        pad[:n] = code
        words = (pad.view(nw, 16) << (2 * torch.arange(16))).sum(1)
        codes.copy_(torch.from_numpy(words.numpy().astype(np.uint32).view(np.int32)))
        return codes
    assert residual.dtype == torch.float32 and residual.numel() == n
    _lib.call("nkb_quant2_flat", g.data_ptr(), int(g.dtype == torch.float32), residual.data_ptr(),
              codes.data_ptr(), n, float(thr), _lib.stream_ptr())
    _lib.count_launch()
    return codes


def dequantize_flat(codes: torch.Tensor, out: torch.Tensor, thr: float, scale: float = 1.0,
                    accumulate: bool = False) -> torch.Tensor:
    n = out.numel()
    if not on_gpu(out):
        w = torch.from_numpy(codes.numpy().view(np.uint32).astype(np.int64))
        c = ((w[:, None] >> (2 * torch.arange(16))) & 3).reshape(-1)[:n]
        val = torch.where(c == 1, thr, torch.where(c == 2, -thr, 0.0)).float() * scale
        flat = out.reshape(-1)
        flat.copy_(((flat.float() + val) if accumulate else val).to(out.dtype))
        return out
    _lib.call("nkb_dequant2_flat", codes.data_ptr(), out.data_ptr(),
              int(out.dtype == torch.float32), n, float(thr), float(scale), int(accumulate),
              _lib.stream_ptr())
    _lib.count_launch()
    return out


def matrix_quantize(A: torch.Tensor, thr: float, R: torch.Tensor | None = None):
    """Returns ``(codes[ceil(n/16), ncol] int32, R)`` for fp32 ``A[n, ncol]``."""
    assert A.dim() == 2 and A.dtype == torch.float32
    n, ncol = A.shape
    m = (n + 15) // 16
    codes = torch.empty(m, ncol, dtype=torch.int32, device=A.device)
    if R is None:
        R = torch.empty_like(A)
    if not on_gpu(A):
        code, res = _codes_cpu(A, thr)
        R.copy_(res)
        pad = torch.zeros(m * 16, ncol, dtype=torch.int64)
        pad[:n] = code
        words = (pad.view(m, 16, ncol) << (2 * torch.arange(16))[None, :, None]).sum(1)
        codes.copy_(torch.from_numpy(words.numpy().astype(np.uint32).view(np.int32)))
        return codes, R
    A = A.contiguous()
    _lib.call("nkb_quant2_matrix", A.data_ptr(), codes.data_ptr(), R.data_ptr(), n, ncol,
              float(thr), _lib.stream_ptr())
    _lib.count_launch()
    return codes, R


def matrix_dequantize(codes: torch.Tensor, n: int, thr: float) -> torch.Tensor:
    m, ncol = codes.shape
    A = torch.empty(n, ncol, dtype=torch.float32, device=codes.device)
    if not on_gpu(codes):
        w = torch.from_numpy(codes.numpy().view(np.uint32).astype(np.int64))
        c = ((w[:, None, :] >> (2 * torch.arange(16))[None, :, None]) & 3).reshape(m * 16, ncol)[:n]
        A.copy_(torch.where(c == 1, thr, torch.where(c == 2, -thr, 0.0)))
        return A
    _lib.call("nkb_dequant2_matrix", A.data_ptr(), codes.data_ptr(), n, ncol, float(thr),
              _lib.stream_ptr())
    _lib.count_launch()
    return A


def _as_tensor(a):
    return torch.from_numpy(a) if isinstance(a, np.ndarray) else a


def cu_fn_matrix_quantize_e(A, C, R, thrd=0.3, bpg=None, tpb=None, to_device=False, stream=None):
    """The reference wrapper's call shape (necklace/cuda/quantize.py:96-115): quantise fp32
    ``A[n, n']`` into the code words ``C[ceil(n/16), n']`` (32-bit) and write the error-feedback
    residual into ``R[n, n']``, all in place.  Tensors or numpy arrays; the launch geometry
    arguments are accepted and unused."""
    a, c, r = _as_tensor(A), _as_tensor(C), _as_tensor(R)
    codes, _ = matrix_quantize(a.contiguous(), float(thrd), r)
    c.view(torch.int32).copy_(codes) if c.dtype != torch.int32 else c.copy_(codes)
    return C


def cu_fn_matrix_dequantize_e(A, C, R=None, thrd=0.3, bpg=None, tpb=None, to_device=False,
                              stream=None):
    """Decode the code words ``C`` into ``A[n, n']`` (+thrd, -thrd or 0 per element), in place
    (necklace/cuda/quantize.py:118-134; ``R`` is not read by the decode)."""
    a, c = _as_tensor(A), _as_tensor(C)
    c32 = c if c.dtype == torch.int32 else c.view(torch.int32)
    a.copy_(matrix_dequantize(c32.contiguous(), a.shape[0], float(thrd)))
    return A
