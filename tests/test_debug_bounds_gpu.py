"""The debug build (TCL_DEBUG_BOUNDS): every possibly-remote data address is checked on the device
before it is used.  A correct run passes unchanged; a plan that is told a wrong range reports
status 9 and skips the accesses - no bad address is ever dereferenced."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

CODE = r"""
import torch
from tileccl_b200 import _build, _native
_build.build(programs=False)
assert _native.lib().tcl_debug_bounds_enabled() == 1
from tileccl_b200.ops.gemm_rs import GemmRs
from tileccl_b200.ops._plan import KernelTimeout
from tileccl_b200.parallel.heap import SymmetricHeap
heap = SymmetricHeap(64 << 20)
A = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16)
Bt = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16)
ref = A.float() @ Bt.float().t()
op = GemmRs(heap, A, Bt, cta_group=2, force_staged=True, timeout_ms=1000)
out = op(); op.check()
assert ((out.float() - ref).abs() / (ref.abs() + 1)).max().item() < 1e-2
print("GOOD_RUN_OK")
# a plan that believes rank 0's memory is 16 bytes long: every staged store must be refused
op2 = GemmRs(heap, A, Bt, cta_group=1, force_staged=True, timeout_ms=300)
op2.plan.lib.tcl_gemm_plan_destroy(op2.plan.handle)
d = op2.plan.desc
d.range_hi[0] = d.range_lo[0] + 16
import ctypes as C
err = C.create_string_buffer(256)
op2.plan.handle = op2.plan.lib.tcl_gemm_plan_create(C.byref(d), err, 256)
op2.stage.zero_()
op2()
try:
    op2.check()
    print("NO_ERROR")
except KernelTimeout as e:
    print("STATUS", e.code)
assert float(op2.stage.abs().max()) == 0.0      # nothing was written through the refused addresses
x = torch.ones(4, device="cuda"); assert float(x.sum()) == 4.0
print("BAD_RANGE_REFUSED")
"""


def test_debug_build_checks_addresses():
    env = dict(os.environ, TILECCL_DEBUG="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", CODE], capture_output=True, text=True, timeout=300, env=env, cwd=root)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "GOOD_RUN_OK" in r.stdout and "STATUS 9" in r.stdout and "BAD_RANGE_REFUSED" in r.stdout
