"""The small- and odd-shape suites once more, on the bounds-checked build of the library.

``libpxe_checked.so`` is the library compiled with -DPXE_BOUNDS_CHECK (include/pxe_debug.h): every global-memory access
of every kernel is looked up in the table of live device allocations first; one that is outside them, crosses the end
of one or is misaligned is skipped and recorded -- nothing traps.  The suites run in a child pytest process (the
library is loaded once per process); tests/conftest.py re-arms the table before every library call and fails a test
whose kernels had an access refused.  Left out: the full-size cases (a binary search per access), the C++ client
(it links libpxe.so itself and allocates outside PyTorch), and the CUDA-graph cases (a table cannot be installed while a stream is being captured).
"""
import ctypes as C
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SUITES = ["test_gpu_epilogue.py", "test_gpu_pool_move.py", "test_gpu_heads.py", "test_gpu_nhwc.py", "test_gpu_guard_zones.py",
          "test_gpu_bn_train.py", "test_gpu_model.py", "test_gpu_graph_parity.py", "test_gpu_vs_reference_cuda.py",
          "test_gpu_torch_spec.py", "test_zz_no_alloc.py"]


def checked_python(code: str) -> subprocess.CompletedProcess:
    return subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True, timeout=600)


@pytest.mark.gpu
def test_checker_sees_an_access_outside_the_table(cuda):
    """Positive control.  With the output left out of the table the kernel's stores are refused -- skipped, not
    performed -- and the report names them; with the input left out its loads yield zeros."""
    code = r"""
import torch
from pixienn_b200 import capi, debug
debug.use_checked_library()
import ctypes as C
x = torch.full((4, 8, 6, 6), 2.0, device="cuda")
y = torch.full_like(x, -7.0)
L = capi.lib()
span = lambda t: (t.data_ptr(), t.numel() * 4)
def run(spans):
    debug.set_allocations(spans)
    fn = debug._plain_lib().pxe_upsample
    capi.check(fn(None, x.data_ptr(), 0, big.data_ptr(), 0, 4, 8, 6, 6, 2, 1.0))
    return debug.read_report()
big = torch.full((4, 8, 12, 12), -7.0, device="cuda")
torch.cuda.synchronize()
rep = run([span(x), span(big)])
assert rep.violations == 0, debug.describe(rep)
assert bool((big == 2.0).all())
big.fill_(-7.0)
rep = run([span(x)])                                   # the output is not in the table
assert rep.violations > 0 and rep.is_store == 1 and rep.file == b"pxe_move.cu" and rep.misaligned == 0, debug.describe(rep)
assert big.data_ptr() <= rep.address < big.data_ptr() + big.numel() * 4
assert bool((big == -7.0).all())                       # every store was skipped
rep = run([span(big)])                                 # the input is not in the table: loads give zeros
assert rep.violations > 0 and rep.is_store == 0, debug.describe(rep)
assert bool((big == 0.0).all())
rep = run([span(x), (big.data_ptr(), big.numel() * 4 - 64)])   # the last 16 outputs lie past the end
assert 0 < rep.violations <= 16, debug.describe(rep)
assert bool((big.flatten()[:-16] == 2.0).all()) and bool((big.flatten()[-16:] == 0.0).all())
print("control ok")
"""
    res = checked_python(code)
    assert res.returncode == 0 and "control ok" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]


@pytest.mark.gpu
def test_suites_on_the_bounds_checked_build(cuda):
    env = dict(os.environ, PXE_TEST_BOUNDS_CHECKED="1")
    cmd = [sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider", "-k", "not pipelined and not cuda_graph and not conv_fusion"] + [os.path.join("tests", s) for s in SUITES]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=3000)
    tail = res.stdout[-3000:] + res.stderr[-2000:]
    assert res.returncode == 0, tail
    m = re.search(r"(\d+) passed", res.stdout)
    assert m and int(m.group(1)) >= 300, tail
