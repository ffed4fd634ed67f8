"""pgb200DmvtNoAlloc - the fused mat-vec pair for callers that cannot allocate
(a program that gave all GPU memory to its own arena, or a latency-critical
section where cudaMalloc/cudaFree would stall the device).

Called straight through the C ABI and compared with pgb200Dmvt, which computes
the same sums with a grown-on-demand workspace.  Two calls in a row share the
library's fixed scratch array, so the second call also shows that what the
first one left behind does no harm.  Collected last (file name), so a run that
stops at the first failure has already run every other test.
"""
import numpy as np
import pytest
import torch

import polygeist_b200 as pgb
from helpers import SEED, elementwise_rel

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
        assert elementwise_rel(x1.cpu().numpy(), r1.cpu().numpy()) <= 1e-12, f"x1, call {call}"
        assert elementwise_rel(x2.cpu().numpy(), r2.cpu().numpy()) <= 1e-12, f"x2, call {call}"
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
