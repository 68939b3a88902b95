"""ctypes binding of the native sm_100a library (``_nkb200.so``).

The library is plain CUDA C++ with a C ABI (see ``csrc/nkb_api.h``): kernels take
raw device pointers and a stream, so binding needs no torch headers and a rebuild
takes seconds.  On a machine with a GPU a missing or unloadable library is an
error (operators never fall back silently to eager PyTorch on CUDA tensors); on
a CPU-only machine the library is optional and operators use their PyTorch
reference implementation for CPU tensors.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
# NKB_DEBUG_BOUNDS=1 selects the bounds-checked debug build (see ``debug_bounds``)
DEBUG_BOUNDS = os.environ.get("NKB_DEBUG_BOUNDS", "0") not in ("", "0")
LIB_PATH = os.path.join(_HERE, "_nkb200_dbg.so" if DEBUG_BOUNDS else "_nkb200.so")

_lock = threading.Lock()
_lib = None
_load_error: Exception | None = None

vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_longlong, C.c_float

_SIGS = {
    "nkb_gemm_bf16": [vp, i64, i32, vp, i64, i32, vp, i64, i32, i32, i32, i32, i32, f32, vp, vp,
                      i64, i32, vp, i64, vp, vp, i32, i32, i32, i32, vp, vp],
    "nkb_norm_fwd": [vp, vp, vp, vp, vp, i32, i32, f32, i32, vp],
    "nkb_norm_bwd_dx": [vp, vp, vp, vp, vp, i32, i32, i32, vp],
    "nkb_norm_bwd_dx_res": [vp, vp, vp, vp, vp, i32, i32, i32, vp, vp],
    "nkb_colsum": [vp, vp, vp, vp, i32, i32, i64, i32, vp],
    "nkb_colsum_fused": [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i64, i32, vp],
    "nkb_f32_to_bf16": [vp, vp, i64, i32, vp],
    "nkb_ce_fwd_bwd": [vp, vp, vp, i32, i32, i64, f32, vp],
    "nkb_ce_stats": [vp, vp, vp, i32, i32, i64, i32, vp],
    "nkb_ce_grad": [vp, vp, vp, i32, i32, i64, i32, f32, vp],
    "nkb_embed_fwd": [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp],
    "nkb_embed_bwd": [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp],
    "nkb_adam_flat": [vp, vp, vp, vp, i32, vp, i64, f32, f32, f32, f32, f32, f32, f32, f32, vp,
                      vp],
    "nkb_hyper_advance": [vp, f32, f32, vp],
    "nkb_sgd_flat": [vp, vp, vp, i32, vp, i64, f32, f32, f32, f32, i32, vp, vp],
    "nkb_clip_coef": [vp, vp, f32, f32, vp],
    "nkb_quant2_flat": [vp, i32, vp, vp, i64, f32, vp],
    "nkb_dequant2_flat": [vp, vp, i32, i64, f32, f32, i32, vp],
    "nkb_quant2_matrix": [vp, vp, vp, i32, i32, f32, vp],
    "nkb_dequant2_matrix": [vp, vp, i32, i32, f32, vp],
    "nkb_scale_cast": [vp, i32, vp, i32, i64, f32, i32, vp],
    "nkb_sumsq": [vp, i32, i64, vp, vp],
    "nkb_attn_fwd": [vp, vp, vp, vp, vp, i32, i32, i32, i32, i64, i64, i64, i64, i64, i64, f32,
                     i32, vp, vp],
    "nkb_attn_bwd": [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i64, i64,
                     i64, i64, i64, i64, f32, i32, vp, vp],
    "nkb_comm_barrier": [vp, i64, i32, i32, vp, vp, vp],
    "nkb_comm_allreduce": [vp, i64, i64, i64, i32, f32, i32, i32, vp, vp, i32, vp],
    "nkb_comm_reduce_scatter": [vp, i64, i64, i64, i32, f32, vp, i32, i32, vp, vp, i32, vp],
    "nkb_comm_bcast": [vp, i64, i64, i64, i32, i32, i32, vp, vp, i32, vp],
    "nkb_comm_allgather": [vp, i64, i64, i64, i32, i32, vp, vp, i32, vp],
    "nkb_comm_dp_quant_allreduce": [vp, i64, vp, i32, vp, i64, i64, vp, i32, i64, f32, f32, i32,
                                    i32, vp, vp, i32, vp],
    "nkb_comm_rs_opt_ag": [vp, i64, i64, i64, i64, vp, vp, vp, i32, f32, f32, f32, f32, f32, f32,
                           f32, f32, i32, vp, i32, i32, vp, vp, i32, vp],
    "nkb_comm_flag_bytes": [],
    "nkb_ag_gemm_bf16": [vp, i64, i64, i32, i32, i32, vp, vp, i32, i64, vp, i64, i32, vp, i64, i32,
                         i32, i32, vp, vp, i64, i32, vp, i64, vp, vp, i32, vp],
    "nkb_gemm_rs_bf16": [vp, i64, i64, i64, i32, i32, i32, vp, vp, i64, vp, i64, i32, vp, i64,
                         i32, i32, vp, vp, i64, vp, i32, vp],
    "nkb_rope": [vp, i32, i32, i32, i32, f32, i32, i32, vp],
    "nkb_swiglu_fwd": [vp, vp, i64, i32, vp],
    "nkb_swiglu_bwd": [vp, vp, vp, i64, i32, vp],
    "nkb_im2col_nhwc": [vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp],
    "nkb_col2im_nhwc": [vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp],
    "nkb_bn_fwd": [vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, f32, f32, i32, vp],
    "nkb_bn_apply": [vp, vp, vp, vp, vp, vp, i64, i32, i32, vp],
    "nkb_bn_bwd": [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, vp, i64, i32, i32, vp],
    "nkb_maxpool3x3s2_fwd": [vp, vp, vp, i32, i32, i32, i32, vp],
    "nkb_maxpool3x3s2_bwd": [vp, vp, vp, i32, i32, i32, i32, vp],
    "nkb_avgpool_fwd": [vp, vp, i32, i32, i32, vp],
    "nkb_avgpool_bwd": [vp, vp, i32, i32, i32, vp],
    "nkb_num_sms": [],
}


class NativeLibraryError(RuntimeError):
    pass


def _try_build() -> None:
    from . import _build
    _build.build(debug_bounds=DEBUG_BOUNDS)


def debug_bounds(raise_on_error: bool = True) -> dict:
    """Debug build only: read and clear the index-check records of every translation unit.
    Returns ``{tu: (count, source line, first bad index)}`` for units with failures and raises
    ``NativeLibraryError`` (device-side error 6, "index check failed") when there are any."""
    lib = load()
    import torch
    torch.cuda.synchronize()
    bad = {}
    for tu in ("conv", "loss", "optim", "comm"):
        fn = getattr(lib, f"nkb_debug_bounds_{tu}", None)
        if fn is None:
            continue
        rec = (C.c_int * 4)()
        fn.argtypes, fn.restype = [C.c_void_p], i32
        check(fn(C.cast(rec, C.c_void_p)), f"nkb_debug_bounds_{tu}")
        if rec[0]:
            bad[tu] = (rec[0], rec[1], (rec[3] << 32) | (rec[2] & 0xffffffff))
    if bad and raise_on_error:
        raise NativeLibraryError(f"device-side error 6 (index check failed): {bad}")
    return bad


def load(build_if_missing: bool = True):
    """Load (building first if needed and possible) and return the ctypes handle."""
    global _lib, _load_error
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        try:
            if not os.path.exists(LIB_PATH) and build_if_missing:
                _try_build()
            lib = C.CDLL(LIB_PATH)
            for name, sig in _SIGS.items():
                fn = getattr(lib, name, None)
                if fn is None:
                    continue  # kernels are added incrementally; absent symbols fail at call time
                fn.argtypes = sig
                fn.restype = i32
            if hasattr(lib, "nkb_build_info"):
                lib.nkb_build_info.restype = C.c_char_p
            _lib = lib
        except Exception as e:  # noqa: BLE001
            _load_error = e
            raise NativeLibraryError(f"cannot load {LIB_PATH}: {e}") from e
    return _lib


def available() -> bool:
    try:
        load()
        return True
    except NativeLibraryError:
        return False


def has(name: str) -> bool:
    return available() and hasattr(_lib, name)


_ERRS = {-1: "cuTensorMapEncodeTiled unavailable", -2: "empty problem", -3: "misaligned operand",
         -4: "size beyond kernel limit", -5: "unsupported configuration"}


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = _ERRS.get(rc, f"cuda error {rc}" if rc > 0 else f"tensor-map/driver error {rc}")
        raise NativeLibraryError(f"{what} failed: {msg}")


def call(name: str, *args) -> None:
    """Call a native entry point, raising on a non-zero return."""
    lib = load()
    fn = getattr(lib, name, None)
    if fn is None:
        raise NativeLibraryError(f"native symbol {name} missing from {LIB_PATH}; rebuild")
    check(fn(*args), name)


def stream_ptr() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


# Count of native kernel launches issued through `call` wrappers that opt in
# (used by bench.py to report how many of this library's kernels ran).
launch_count = 0


def count_launch(n: int = 1) -> None:
    global launch_count
    launch_count += n
