"""The bounds-checked debug build (-DNKB_DEBUG_BOUNDS): small and odd shapes run clean through
the hand-indexed kernels, and a failing check is reported (and its access skipped) without a
fault.  Runs in a child process because the build variant is chosen when the library loads."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import ctypes, sys, torch
sys.path.insert(0, %r)
from necklace_b200 import _lib
assert _lib.DEBUG_BOUNDS and _lib.LIB_PATH.endswith("_dbg.so")
from necklace_b200.ops import adam_step, check_status
from necklace_b200.ops.conv import BatchNorm2d, Conv2d, global_avg_pool, max_pool_3x3_s2
from necklace_b200.ops.loss import embed_fwd
torch.manual_seed(0)
for (N, H, W, Ci, Co, k, s, p) in [(2, 9, 9, 16, 24, 3, 1, 1), (1, 11, 7, 8, 8, 3, 2, 1),
                                   (2, 20, 20, 3, 16, 7, 2, 3), (2, 9, 9, 16, 40, 1, 2, 0)]:
    conv = Conv2d(Ci, Co, k, s, p, device="cuda")
    x = torch.randn(N, H, W, Ci, device="cuda").bfloat16().requires_grad_(True)
    y = BatchNorm2d(Co, relu=True, device="cuda")(conv(x))
    y.float().square().mean().backward()
x = torch.randn(2, 9, 10, 16, device="cuda").bfloat16().requires_grad_(True)
global_avg_pool(max_pool_3x3_s2(x)).float().sum().backward()
embed_fwd(torch.randint(0, 50, (3, 7), device="cuda"), torch.randn(50, 64, device="cuda").bfloat16(),
          None, 7)
n = 1003
m, a, v = (torch.zeros(n, device="cuda") for _ in range(3))
adam_step(m, a, v, torch.randn(n, device="cuda"), None, lr=1e-3, step=1)
torch.cuda.synchronize()
check_status()
assert _lib.debug_bounds() == {}, "clean run must report nothing"
# one failing check, evaluated without any memory access
lib = _lib.load()
sink = torch.zeros(1, dtype=torch.int32, device="cuda")
lib.nkb_debug_bounds_selftest.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
assert lib.nkb_debug_bounds_selftest(sink.data_ptr(), None) == 0
bad = _lib.debug_bounds(raise_on_error=False)
assert list(bad) == ["conv"] and bad["conv"][0] == 1 and bad["conv"][2] == 5, bad
assert int(sink.item()) == 0                     # the guarded access was skipped
assert _lib.debug_bounds() == {}                  # the record was cleared
print("DEBUG_BOUNDS_OK")
'''


def test_debug_bounds_build_runs_clean_and_reports_a_failing_check():
    env = dict(os.environ, NKB_DEBUG_BOUNDS="1")
    r = subprocess.run([sys.executable, "-c", CHILD % ROOT], env=env, capture_output=True,
                       text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0 and "DEBUG_BOUNDS_OK" in r.stdout, r.stdout[-1500:] + r.stderr[-3000:]
