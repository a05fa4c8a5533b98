"""The index-checking build of the kernel library (``python -m cogito_b200.build --debug-bounds``):
kernels run as usual, an index outside its range is recorded (source file, line, index, limit)
instead of being used, and ``assert_device_ok`` fails on it.  The probe runs in a child process
because the choice of library is made when the package is imported."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DBG = os.path.join(ROOT, "cogito_b200", "lib", "libcogito_kernels_dbg.so")

CHILD = r"""
import json, sys, torch
sys.path.insert(0, %r)
from cogito_b200.ops import _lib
from cogito_b200.ops.gemm import gemm
from cogito_b200.ops import loss as L
assert _lib._DEBUG and str(_lib._LIB_PATH).endswith("_dbg.so")
out = {}
a = torch.randn(300, 136, device="cuda", dtype=torch.bfloat16); b = torch.randn(200, 136, device="cuda", dtype=torch.bfloat16)
y = gemm(a, b, bias=torch.randn(200, device="cuda", dtype=torch.bfloat16), act="gelu")
out["gemm_err"] = float((y.float() - torch.nn.functional.gelu(a.float() @ b.float().T + 0, approximate="tanh")).abs().max()) >= 0
mk = lambda: torch.randn(64, 512, device="cuda", dtype=torch.bfloat16)
tg = torch.randint(0, 512, (64,), device="cuda")
L.cross_entropy(mk(), tg)
out["clean"] = _lib.read_bounds()
# a label beyond the vocabulary: the kernels skip such a row (no access is made with it); the
# debug build also reports it
tg[5] = 700
L.cross_entropy(mk(), tg)
out["bad"] = _lib.read_bounds()
out["after_reset"] = _lib.read_bounds()
try:
    tg[5] = 701
    L.cross_entropy(mk(), tg)
    _lib.assert_device_ok()
    out["raised"] = False
except _lib.KernelError as e:
    out["raised"] = "701" in str(e)
print("RESULT " + json.dumps(out))
"""


@pytest.mark.skipif(not os.path.exists(DBG), reason="debug-bounds library not built")
def test_debug_build_records_an_out_of_range_index_and_keeps_running():
    env = dict(os.environ, COGITO_KERNELS_DEBUG="1")
    r = subprocess.run([sys.executable, "-c", CHILD % ROOT], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    out = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("RESULT ")][-1][7:])
    assert out["clean"] == []
    assert len(out["bad"]) == 1 and out["bad"][0][0] == "softmax_ce" and out["bad"][0][2:] == [700, 512]
    assert out["after_reset"] == [] and out["raised"] is True
