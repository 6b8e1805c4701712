"""The checking build of the kernel library (``AERIS_BOUNDS_CHECK=1``: every gather-table entry and push owner is
validated on the device; a bad one is recorded in the status word and the access is skipped, never trapped) stands in
for a memory checker. It runs in a child process because the choice of library is made at import time."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import sys, torch
sys.path.insert(0, %r)
from aeris_gb_b200.ops import elementwise as E, lib as L
from aeris_gb_b200.ops.build import CHECKED, LIB_PATH
assert CHECKED and LIB_PATH.name == "libaeris_b200_chk.so"
dev = "cuda"
D, rows = 256, 64
# the source buffer is larger than the 64 rows declared to the check, so even an unchecked access would stay inside it
src = torch.randn(2 * rows, D, device=dev).bfloat16()
table = torch.arange(rows, device=dev, dtype=torch.int32)
out = torch.empty(rows, D, device=dev, dtype=torch.bfloat16)
assert E.set_gather_bounds(rows)
E.gather_rows(table, [src.data_ptr()], out, src_rows=rows)
L.check_status()
assert torch.equal(out, src[:rows])
bad = table.clone(); bad[5] = rows + 17            # beyond the declared rows
E.gather_rows(bad, [src.data_ptr()], out, src_rows=rows)
try:
    L.check_status()
    raise SystemExit("a gather code beyond the source rows was not reported")
except L.KernelError as e:
    assert "bounds" in str(e)
assert float(out[5].float().abs().max()) == 0.0 and torch.equal(out[6], src[6])
bad2 = table.clone(); bad2[9] = (3 << 28) | 2      # a rank that has no buffer
E.gather_rows(bad2, [src.data_ptr()], out, src_rows=rows)
try:
    L.check_status()
    raise SystemExit("a gather code naming a missing rank was not reported")
except L.KernelError:
    pass
# the same through the fused modulate+norm gather
w = torch.ones(D, device=dev).bfloat16()
h = torch.empty(rows, D, device=dev, dtype=torch.bfloat16); xo = torch.empty_like(h)
E.modnorm_fwd(None, None, None, w, mode=1, eps=1e-3, out=h, gather_idx=bad, peer_ptrs=[src.data_ptr()], x_out=xo, rows=rows,
              src_rows=rows)
try:
    L.check_status()
    raise SystemExit("modnorm gather did not report")
except L.KernelError:
    pass
E.modnorm_fwd(None, None, None, w, mode=1, eps=1e-3, out=h, gather_idx=table, peer_ptrs=[src.data_ptr()], x_out=xo, rows=rows,
              src_rows=rows)
L.check_status()
assert torch.equal(xo, src[:rows])
print("checked build ok")
''' % ROOT


def test_checked_build_reports_bad_gather_codes_and_skips_them():
    env = dict(os.environ, AERIS_BOUNDS_CHECK="1")
    r = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0 and "checked build ok" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


def test_kernel_and_model_tests_pass_on_the_checked_build():
    """The block-level tests (gather tables of the shifted layers, regroup, push-free paths) once more on the checking
    library: no table entry of a real run may trip a check."""
    env = dict(os.environ, AERIS_BOUNDS_CHECK="1")
    r = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu", "tests/test_model_gpu.py", "-k",
                        "matches_oracle"], capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
