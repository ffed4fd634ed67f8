"""pgb200DmvtNoAlloc - the fused mat-vec pair for callers that cannot allocate
(a program that gave all GPU memory to its own arena, or a latency-critical
section where cudaMalloc/cudaFree would stall the device).

Called straight through the C ABI and compared with pgb200Dmvt, which computes
the same sums with a grown-on-demand workspace.  Two calls in a row share the
library's fixed scratch array, so the second call also shows that what the
first one left behind does no harm.  Collected last (file name), so a run that
stops at the first failure has already run every other test.
"""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import polygeist_b200 as pgb
from helpers import SEED

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _filled(shape, aid):
    t = torch.empty(shape, dtype=torch.float64, device=DEV)
    pgb.fill_uniform(t, SEED, aid, 0.0, 1.0)
    return t


def _pair(n, lda_pad, aid0):
    buf = _filled((n, n + lda_pad), aid0)
    A = buf[:, :n]
    vec = [_filled((n,), aid0 + 1 + k) for k in range(4)]  # x1, x2, y1, y2
    return A, vec


@pytest.mark.parametrize("n,pad", [(1000, 0), (4096, 0), (333, 3)])
def test_no_alloc_matches_dmvt_on_two_calls_in_a_row(n, pad):
    lib = pgb.load()
    stream = torch.cuda.current_stream().cuda_stream
    for call, aid0 in enumerate((10, 20)):  # second call: new data, same static scratch
        A, (x1, x2, y1, y2) = _pair(n, pad, aid0)
        r1, r2 = x1.clone(), x2.clone()
        st = lib.pgb200Dmvt(stream, n, A.data_ptr(), n + pad, y1.data_ptr(), y2.data_ptr(),
                            r1.data_ptr(), r2.data_ptr())
        assert st == pgb.OK
        st = lib.pgb200DmvtNoAlloc(stream, n, A.data_ptr(), n + pad, y1.data_ptr(), y2.data_ptr(),
                                   x1.data_ptr(), x2.data_ptr())
        assert st == pgb.OK, lib.pgb200GetLastErrorString()
        torch.cuda.synchronize()
        # Same first pass, same second pass: the two entry points agree bit for bit.
        assert np.array_equal(x1.cpu().numpy(), r1.cpu().numpy()), f"x1, call {call}"
        assert np.array_equal(x2.cpu().numpy(), r2.cpu().numpy()), f"x2, call {call}"
        # and the pair itself is right, not merely equal: x1 - x1_before == A @ y1
        A64 = A.cpu().numpy()
        assert np.allclose(r1.cpu().numpy(), _filled((n,), aid0 + 1).cpu().numpy() + A64 @ y1.cpu().numpy(),
                           rtol=1e-12, atol=0)


def test_no_alloc_rejects_what_it_cannot_serve():
    lib = pgb.load()
    n = 4097
    d = torch.zeros(8, dtype=torch.float64, device=DEV)
    p = d.data_ptr()
    assert lib.pgb200DmvtNoAlloc(None, n, p, n, p, p, p, p) == pgb.ERR_INVALID
    assert b"4096" in lib.pgb200GetLastErrorString()
    h = np.zeros((4, 4))
    v = np.zeros(4)
    assert lib.pgb200DmvtNoAlloc(None, 4, h.ctypes.data, 4, v.ctypes.data, v.ctypes.data,
                                 v.ctypes.data, v.ctypes.data) == pgb.ERR_INVALID
    assert lib.pgb200DmvtNoAlloc(None, 0, None, 0, None, None, None, None) == pgb.OK


def test_no_alloc_reserves_no_device_memory():
    """Free device memory reads the same before and after calls (the first call
    has already looked the array's address up, which reserves nothing either)."""
    lib = pgb.load()
    n = 2048
    A, (x1, x2, y1, y2) = _pair(n, 0, 30)
    stream = torch.cuda.current_stream().cuda_stream
    args = (stream, n, A.data_ptr(), n, y1.data_ptr(), y2.data_ptr(), x1.data_ptr(), x2.data_ptr())
    assert lib.pgb200DmvtNoAlloc(*args) == pgb.OK
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        assert lib.pgb200DmvtNoAlloc(*args) == pgb.OK
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0


_FIRST_CALL = r"""
import ctypes as C, sys
import numpy as np
import torch
sys.path.insert(0, sys.argv[1])
import polygeist_b200 as pgb
lib = pgb.load()            # loads the library; no entry point has been called yet
n = 777
g = torch.Generator(device="cuda").manual_seed(1)
A = torch.rand((n, n), dtype=torch.float64, device="cuda", generator=g)
v = [torch.rand(n, dtype=torch.float64, device="cuda", generator=g) for _ in range(4)]
x1, x2, y1, y2 = v
e1, e2 = x1 + A @ y1, x2 + A.T @ y2
torch.cuda.synchronize()
st = lib.pgb200DmvtNoAlloc(None, n, A.data_ptr(), n, y1.data_ptr(), y2.data_ptr(),
                           x1.data_ptr(), x2.data_ptr())
torch.cuda.synchronize()
assert st == 0, lib.pgb200GetLastErrorString()
assert torch.allclose(x1, e1, rtol=1e-12, atol=0) and torch.allclose(x2, e2, rtol=1e-12, atol=0)
# The library image (code and the fixed array) is on the device now; from here
# on a call must leave the amount of free device memory unchanged.
free0, _ = torch.cuda.mem_get_info()
st = lib.pgb200DmvtNoAlloc(None, n, A.data_ptr(), n, y1.data_ptr(), y2.data_ptr(),
                           x1.data_ptr(), x2.data_ptr())
torch.cuda.synchronize()
free1, _ = torch.cuda.mem_get_info()
assert st == 0 and free1 == free0, (st, free0, free1)
print("first-call-ok")
"""


def test_no_alloc_works_as_the_first_library_call_of_a_process():
    """Nothing else has initialised the library's runtime: the entry point must
    stand on its own; once the library image is resident, a further call leaves
    the free device memory unchanged."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", _FIRST_CALL, root], capture_output=True, text=True,
                         timeout=300)
    assert out.returncode == 0 and "first-call-ok" in out.stdout, out.stdout + out.stderr
