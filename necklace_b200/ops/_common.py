"""Shared helpers for the operator wrappers."""
from __future__ import annotations

import torch

from .. import _lib

_status: dict[int, torch.Tensor] = {}
_scratch: dict[tuple, torch.Tensor] = {}

STATUS_TEXT = {
    0: "ok", 1: "MMA warp timed out waiting for a TMA stage",
    2: "TMA producer timed out waiting for a free stage",
    3: "epilogue timed out waiting for an accumulator",
    4: "MMA warp timed out waiting for a free accumulator",
    5: "timed out waiting for a readiness/peer flag", 6: "index check failed",
}


def on_gpu(*ts) -> bool:
    """True when the native path must be used (any CUDA tensor)."""
    return any(t is not None and t.is_cuda for t in ts)


def status_word(device=None) -> torch.Tensor:
    """Device int32 the kernels write their first error code to."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    t = _status.get(dev)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=f"cuda:{dev}")
        _status[dev] = t
    return t


def check_status(reset: bool = True) -> None:
    """Synchronise and raise if any kernel since the last check reported an error."""
    for dev, t in _status.items():
        code = int(t.item())
        if code != 0:
            if reset:
                t.zero_()
            raise _lib.NativeLibraryError(
                f"device-side error {code} on cuda:{dev}: {STATUS_TEXT.get(code, 'unknown')}")


def scratch(key: str, numel: int, dtype: torch.dtype, device) -> torch.Tensor:
    """A cached scratch tensor per (key, device); grown, never shrunk."""
    k = (key, str(device), dtype)
    t = _scratch.get(k)
    if t is None or t.numel() < numel:
        t = torch.empty(max(numel, 1), dtype=dtype, device=device)
        _scratch[k] = t
    return t[:numel]


def scratch_zero(key: str, numel: int, dtype: torch.dtype, device) -> torch.Tensor:
    """Like ``scratch`` but zero-filled when (re)allocated; for kernels that leave their
    scratch at zero on exit (accumulators, ticket counters)."""
    k = (key, str(device), dtype, "z")
    t = _scratch.get(k)
    if t is None or t.numel() < numel:
        t = torch.zeros(max(numel, 1), dtype=dtype, device=device)
        _scratch[k] = t
    return t


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def set_wait_cycles(cycles: int) -> None:
    """Limit (in SM clock cycles) of every bounded device-side wait: on a barrier, on a peer
    flag, on a readiness flag.  The default is about two seconds; a wait that runs out makes
    its kernel record a status code and return (see ``check_status``)."""
    lib = _lib.load()
    for tu in ("gemm", "attn", "comm"):
        fn = getattr(lib, f"nkb_set_wait_cycles_{tu}")
        fn.argtypes = [_lib.i64]
        fn.restype = _lib.i32
        _lib.check(fn(int(cycles)), f"nkb_set_wait_cycles_{tu}")
