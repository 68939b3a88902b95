"""Assorted PyTorch helpers (reference: necklace/frmwrk/pytorch/ptutils.py:11-222)."""
from __future__ import annotations

import gc
from collections import OrderedDict

import torch


def pt_dtype_to_str(dtype):
    return str(dtype).split(".")[-1]


def clip_grad_norm(model, clip=0.25, *args, **kwargs):
    return torch.nn.utils.clip_grad_norm_(model.parameters(), clip, *args, **kwargs)


def get_state_dict_from_dp(pth_tar, state_key="state_dict"):
    """Load a checkpoint saved from a ``DataParallel`` model: strips the ``module.`` prefix.
    ``pth_tar`` is a path or an already loaded dict."""
    ckpt = torch.load(pth_tar, map_location="cpu") if isinstance(pth_tar, str) else pth_tar
    sd = ckpt[state_key] if state_key and state_key in ckpt else ckpt
    out = OrderedDict()
    for k, v in sd.items():
        out[k[7:] if k.startswith("module.") else k] = v
    return out


def get_param_size(model):
    return sum(p.numel() for p in model.parameters())


def prnt_md(model):
    """Print a table of parameter names, shapes and sizes; returns the total count."""
    rows = [(n, tuple(p.shape), p.numel()) for n, p in model.named_parameters()]
    w = max((len(r[0]) for r in rows), default=4)
    for n, s, c in rows:
        print(f"{n:<{w}}  {str(s):<24} {c:>12,d}")
    total = sum(r[2] for r in rows)
    print(f"{'total':<{w}}  {'':<24} {total:>12,d}")
    return total


def clear_tensor_mem(t=None, do_gc=False, do_pt_cache=True):
    del t
    if do_gc:
        gc.collect()
    if do_pt_cache and torch.cuda.is_available():
        torch.cuda.empty_cache()


def _mb(x):
    return round(x / (1024 * 1024), 2)


def see_memory_usage(message, force=False):
    if not force or not torch.cuda.is_available():
        return None
    s = {"allocated_mb": _mb(torch.cuda.memory_allocated()),
         "max_allocated_mb": _mb(torch.cuda.max_memory_allocated()),
         "reserved_mb": _mb(torch.cuda.memory_reserved())}
    print(message, s)
    return s


show_cuda_memory_usage = see_memory_usage


class PtCudaMemUsage:
    """Absolute and delta memory report between calls."""

    def __init__(self, do_print=True):
        self.do_print, self.last = do_print, 0

    def show(self, msg=""):
        cur = torch.cuda.memory_allocated() if torch.cuda.is_available() else 0
        out = {"allocated_mb": _mb(cur), "delta_mb": _mb(cur - self.last)}
        self.last = cur
        if self.do_print:
            print("[mem]", msg, out)
        return out


def memory_status(msg, print_rank=-1, reset_max=False):
    if not torch.cuda.is_available():
        return None
    s = {"alloc": _mb(torch.cuda.memory_allocated()), "max_alloc": _mb(torch.cuda.max_memory_allocated()),
         "cache": _mb(torch.cuda.memory_reserved()), "max_cache": _mb(torch.cuda.max_memory_reserved())}
    if reset_max:
        torch.cuda.reset_peak_memory_stats()
    print("memory_status", msg, s)
    return s


def get_ma_status():
    return torch.cuda.memory_allocated() if torch.cuda.is_available() else 0


def pad_line(aj, mxs):
    """Cells of one row padded with blanks to the column widths ``mxs``."""
    return [c + " " * (w - len(c)) for c, w in zip(aj, mxs)]


def prnt_by_tab(a):
    """Print rows of strings as a table: columns padded to their widest cell, joined by tabs
    (reference: necklace/frmwrk/pytorch/ptutils.py:65-81)."""
    if not a:
        return
    mxs = [max(len(row[i]) for row in a) for i in range(len(a[0]))]
    for row in a:
        print("\t".join(pad_line(row, mxs)))
