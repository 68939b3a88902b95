"""The allocation-free column-sum entry point against the regular one (GPU).

Some users of this library must not allocate device memory when they call it (a
host application that has handed out all GPU memory up front, or code running while
the allocator is frozen), so ``nkb_colsum_bf16_noalloc`` keeps its fp32 accumulator
in a static device array inside the library.  The test calls it through the exported
C symbol, exactly as such a caller would, twice in a row with different data (the
scratch is shared and keeps old contents, so the second call checks the clearing),
and compares with the regular path that uses caller-allocated scratch.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _noalloc_fn():
    from necklace_b200 import _lib
    lib = _lib.load()
    fn = lib.nkb_colsum_bf16_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                   ctypes.c_longlong, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return fn


def test_noalloc_colsum_matches_regular_entry_point_twice():
    from necklace_b200.ops.gemm import colsum
    fn = _noalloc_fn()
    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    for rows, C, scale in [(4096, 1024, 1.0), (1000, 3072, -3.0)]:
        dy = (torch.randn(rows, C, device="cuda") * scale).bfloat16()
        out = torch.full((C,), 123.0, device="cuda", dtype=torch.bfloat16)
        before = torch.cuda.memory_allocated()
        rc = fn(dy.data_ptr(), out.data_ptr(), rows, C, dy.stride(0), stream)
        assert rc == 0
        assert torch.cuda.memory_allocated() == before  # nothing came from the torch allocator
        ref = colsum(dy)
        torch.cuda.synchronize()
        err = ((out.float() - ref.float()).norm() / (ref.float().norm() + 1e-12)).item()
        assert err < 1e-2, err
        exact = dy.float().sum(0)
        assert ((out.float() - exact).norm() / exact.norm()).item() < 1e-2


def test_noalloc_rejects_oversize_and_odd():
    fn = _noalloc_fn()
    x = torch.zeros(2, 8, device="cuda", dtype=torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream
    assert fn(x.data_ptr(), x.data_ptr(), 2, 65536 + 2, 65538, stream) == -4
    assert fn(x.data_ptr(), x.data_ptr(), 2, 7, 8, stream) == -3
