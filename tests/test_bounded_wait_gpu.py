"""Device-side waits are bounded: a flag that nothing sets makes the kernel give up,
record a status code and return; the host raises and the context stays usable."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_gemm_readiness_flag_timeout_reports_status_and_context_survives():
    from necklace_b200 import _lib
    from necklace_b200.ops import check_status, gemm
    from necklace_b200.ops._common import set_wait_cycles
    A = torch.randn(256, 128, device="cuda").bfloat16()
    B = torch.randn(256, 128, device="cuda").bfloat16()
    flags = torch.zeros(2, dtype=torch.int32, device="cuda")  # never raised to the target
    set_wait_cycles(20_000_000)          # about 10 ms instead of the default two seconds
    try:
        gemm(A, B, ready_flags=flags, rows_per_flag=128, ready_target=1, bn=256)
        with pytest.raises(_lib.NativeLibraryError, match="flag"):
            check_status()
    finally:
        set_wait_cycles(4_000_000_000)
    # the context is intact: the same call succeeds once the flags are set
    flags.fill_(1)
    out = gemm(A, B, ready_flags=flags, rows_per_flag=128, ready_target=1, bn=256)
    check_status()
    ref = A.float() @ B.float().t()
    assert ((out.float() - ref).norm() / ref.norm()).item() < 1e-2
