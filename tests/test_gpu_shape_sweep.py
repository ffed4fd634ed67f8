"""Shape sweep of the GEMM and rank-k entry points against the CPU oracle.

compute-sanitizer is closed on the GPU pool, so out-of-bounds accesses are
looked for the way a caller would meet them: every output array is embedded in
a larger NaN-filled buffer (canary rows below and columns to the right), the
operands have randomly padded leading dimensions and sit at randomly
misaligned offsets, and after each call the canaries must still be NaN and the
result must match the loop nest.  Extents are drawn from the edges of the tile
sizes (1, 2, 3, 5, 8, 15..17, 31..33, 63..65, 127..129, 255..257) with a few long
K that reach the split-K and chunked-accumulation paths.
"""
import numpy as np
import pytest
import torch

import polygeist_b200 as pgb
from helpers import SEED, elementwise_rel
from oracle import pbo

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
EDGES = [1, 2, 3, 5, 8, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 256, 257]
LONG_K = [384, 512, 1000, 1024, 2048, 2050]


def _embedded(rows, cols, dtype, rng, aid, lo, hi, canary_rows=0):
    """A rows x cols operand inside a NaN-filled buffer: random extra leading
    dimension, random element offset of the first entry (so bases are not always
    16-byte aligned), `canary_rows` rows below.  Returns (view, whole buffer)."""
    pad = int(rng.integers(0, 4))
    off = int(rng.integers(0, 4))
    ld = cols + pad
    buf = torch.full(((rows + canary_rows) * ld + off + 8,), float("nan"), dtype=dtype, device=DEV)
    view = buf[off:off + rows * ld].view(rows, ld)[:, :cols]
    pgb.fill_uniform(view, SEED, aid, lo, hi)
    return view, buf


def _canaries_intact(buf, view, rows, cols):
    """Everything of `buf` outside the rows x cols window is still NaN."""
    mask = torch.ones_like(buf, dtype=torch.bool)
    ld = view.stride(0) if rows > 1 else cols
    off = view.storage_offset() - buf.storage_offset()
    idx = (off + torch.arange(rows, device=DEV)[:, None] * ld + torch.arange(cols, device=DEV)[None, :])
    mask[idx.reshape(-1)] = False
    return bool(torch.isnan(buf[mask]).all())


def _shapes(seed, count):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(count):
        M, N = int(rng.choice(EDGES)), int(rng.choice(EDGES))
        K = int(rng.choice(LONG_K)) if i % 4 == 0 else int(rng.choice(EDGES))
        out.append((M, N, K, float(rng.choice([0.0, 1.2]))))
    return out


@pytest.mark.parametrize("dtype,np_dtype,lo", [(torch.float64, np.float64, -1.0),
                                               (torch.float32, np.float32, 0.0)])
def test_gemm_shape_sweep_with_canaries(dtype, np_dtype, lo):
    rng = np.random.default_rng(SEED + (1 if dtype == torch.float64 else 2))
    worst = 0.0
    for n, (M, N, K, beta) in enumerate(_shapes(SEED + 7, 160)):
        A, _ = _embedded(M, K, dtype, rng, 1, lo, 1.0)
        B, _ = _embedded(K, N, dtype, rng, 2, lo, 1.0)
        Cm, cbuf = _embedded(M, N, dtype, rng, 3, lo, 1.0, canary_rows=2)
        hA, hB, hC = (np.ascontiguousarray(t.cpu().numpy()) for t in (A, B, Cm))
        if beta == 0.0:
            Cm.fill_(float("nan"))      # beta == 0 must not read C
        pgb.gemm(1.5, A, B, beta, Cm)
        torch.cuda.synchronize()
        pgb.poll_device_status()
        got = Cm.cpu().numpy()
        where = f"case {n}: M={M} N={N} K={K} beta={beta} lda={A.stride(0)} ldb={B.stride(0)} ldc={Cm.stride(0)}"
        assert _canaries_intact(cbuf, Cm, M, N), "wrote outside C, " + where
        if np_dtype == np.float64:
            ref = pbo.gemm(1.5, beta, hC.copy(), hA, hB)
            # normwise, with a floor on the scale: a 1 x 1 result of signed data can be ~0
            err = float(np.max(np.abs(got - ref)) / max(np.max(np.abs(ref)), 1.0))
            assert err <= 1e-12, where
        else:
            truth = pbo.gemm_acc64(1.5, beta, hC, hA, hB)
            err = elementwise_rel(got, truth)
            assert err <= 1e-5, where
        worst = max(worst, err)
    assert worst > 0.0      # the sweep really compared different summation orders


@pytest.mark.parametrize("dtype,np_dtype,lo", [(torch.float64, np.float64, -1.0),
                                               (torch.float32, np.float32, 0.0)])
def test_syrk_shape_sweep_with_canaries(dtype, np_dtype, lo):
    rng = np.random.default_rng(SEED + 11)
    for n_case in range(60):
        n = int(rng.choice(EDGES + [300, 513]))
        k = int(rng.choice(LONG_K)) if n_case % 3 == 0 else int(rng.choice(EDGES))
        A, _ = _embedded(n, k, dtype, rng, 1, lo, 1.0)
        Cm, cbuf = _embedded(n, n, dtype, rng, 2, lo, 1.0, canary_rows=2)
        hA, hC = (np.ascontiguousarray(t.cpu().numpy()) for t in (A, Cm))
        pgb.syrk(1.5, A, 1.2, Cm)
        torch.cuda.synchronize()
        pgb.poll_device_status()
        got = Cm.cpu().numpy()
        where = f"case {n_case}: n={n} k={k} lda={A.stride(0)} ldc={Cm.stride(0)}"
        assert _canaries_intact(cbuf, Cm, n, n), "wrote outside C, " + where
        il, iu = np.tril_indices(n), np.triu_indices(n, 1)
        assert np.array_equal(got[iu], hC[iu]), "strict upper triangle touched, " + where
        if np_dtype == np.float64:
            ref = pbo.syrk(1.5, 1.2, hC.copy(), hA)
            assert float(np.max(np.abs(got[il] - ref[il])) / max(np.max(np.abs(ref[il])), 1.0)) <= 1e-12, where
        else:
            truth = 1.5 * (hA.astype(np.float64) @ hA.astype(np.float64).T) + 1.2 * hC.astype(np.float64)
            assert elementwise_rel(got[il], truth[il]) <= 1e-5, where
