"""GPU parity tests: every call goes through the C ABI of libpgb200 and is
checked against the CPU oracle on the same seeded inputs.

Gates (the tolerances BASELINE.json states, made precise):
  fp64, signed inputs  : max|d| / max|ref| <= 1e-12, and componentwise backward
                         error |d| / (|a||A||B| + |b||C|) <= 1e-13
  fp64, inputs in [0,1): element-wise relative error <= 1e-12
  fp32                 : element-wise relative error <= 1e-5 against the fp64-
                         accumulated evaluation of the same fp32 inputs, and
                         against the sequential fp32 loop nest where K <= 8192
"""
import numpy as np
import pytest
import torch

import polygeist_b200 as pgb
from helpers import (MINI, SEED, assert_dump_equal, backward_gemm, elementwise_rel, init_2mm,
                     init_3mm, init_atax, init_bicg, init_gemm, init_gemver, init_gesummv, init_mvt,
                     init_doitgen, init_symm, init_syr2k, init_syrk, init_trmm,
                     normwise, read_dump)
from oracle import pbo
from polygeist_b200 import polybench

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev_fill(rows, cols, dtype, aid, lo, hi, ld=None):
    ld = cols if ld is None else ld
    buf = torch.full((rows, ld), float("nan"), dtype=dtype, device=DEV)
    view = buf[:, :cols]
    pgb.fill_uniform(view, SEED, aid, lo, hi)
    return view


def sync_ok():
    torch.cuda.synchronize()
    pgb.poll_device_status()


# --------------------------------------------------------------------------- generator
@pytest.mark.parametrize("dtype,np_dtype", [(torch.float64, np.float64), (torch.float32, np.float32)])
def test_device_generator_is_bit_identical_to_host(dtype, np_dtype):
    d = dev_fill(33, 47, dtype, 3, -1.0, 1.0, ld=52)
    h = pbo.fill(33, 47, np_dtype, SEED, 3, -1.0, 1.0)
    assert np.array_equal(d.cpu().numpy(), h)
    part = torch.empty((5, 47), dtype=dtype, device=DEV)
    pgb.fill_uniform(part, SEED, 3, -1.0, 1.0, row0=11)
    assert np.array_equal(part.cpu().numpy(), h[11:16])


# --------------------------------------------------------------------------- dgemm
DGEMM_SHAPES = [
    # (M, N, K, lda_pad, ldb_pad, ldc_pad, expect fast path)
    (128, 128, 64, 0, 0, 0, True),
    (256, 384, 512, 0, 0, 0, True),
    (200, 152, 100, 0, 0, 0, True),      # ragged tiles, K not a multiple of 16
    (1, 4, 4, 0, 0, 0, True),
    (130, 260, 36, 6, 2, 4, True),       # padded leading dimensions
    (97, 61, 45, 0, 0, 0, True),         # odd sizes: repacked with a padded inner extent
    (64, 64, 64, 1, 0, 0, True),         # odd lda: A repacked
    (64, 66, 64, 0, 1, 0, True),         # odd ldb, N not a multiple of 4: B repacked
    (17, 33, 1, 0, 0, 0, True),
    (1001, 1003, 1005, 0, 0, 0, True),
]


@pytest.mark.parametrize("M,N,K,pa,pb,pc,fast", DGEMM_SHAPES)
@pytest.mark.parametrize("beta", [1.2, 0.0])
def test_dgemm_matches_oracle(M, N, K, pa, pb, pc, fast, beta):
    A = dev_fill(M, K, torch.float64, 1, -1.0, 1.0, ld=K + pa)
    B = dev_fill(K, N, torch.float64, 2, -1.0, 1.0, ld=N + pb)
    Cm = dev_fill(M, N, torch.float64, 3, -1.0, 1.0, ld=N + pc)
    hA, hB, hC = A.cpu().numpy(), B.cpu().numpy(), Cm.cpu().numpy()
    C0 = hC.copy()
    if beta == 0.0:
        Cm.fill_(float("nan"))  # beta == 0 must not read C
    pgb.gemm(1.5, A, B, beta, Cm)
    sync_ok()
    assert pgb.last_path() == (pgb.PATH_DMMA if fast else pgb.PATH_SIMT)
    if M == 1001 and beta == 0.0:
        return  # the oracle run of this size is made once, with beta != 0
    ref = pbo.gemm(1.5, beta, np.ascontiguousarray(hC), np.ascontiguousarray(hA),
                   np.ascontiguousarray(hB))
    got = Cm.cpu().numpy()
    assert normwise(got, ref) <= 1e-12
    assert backward_gemm(got, ref, 1.5, beta, hA, hB, C0) <= 1e-13
    if pc:
        assert torch.isnan(Cm._base[:, N:]).all(), "padding columns must keep their NaN fill"


@pytest.mark.parametrize("M,N,K,beta", [(512, 512, 512, 1.2), (1000, 1100, 1200, 1.2),
                                         (256, 384, 4096, 0.0), (130, 252, 1028, 1.2)])
def test_dgemm_split_k(M, N, K, beta):
    """Few tiles: the K-blocks of every tile are dealt to several CTAs and the
    partial products added in split order (two launches).  Checked against the
    loop nest, for bit-identical repeats, and against the unsplit kernel."""
    A = dev_fill(M, K, torch.float64, 1, -1.0, 1.0)
    B = dev_fill(K, N, torch.float64, 2, -1.0, 1.0)
    C0 = dev_fill(M, N, torch.float64, 3, -1.0, 1.0)
    hA, hB, hC = (np.ascontiguousarray(t.cpu().numpy()) for t in (A, B, C0))

    def run():
        Cm = C0.clone() if beta != 0.0 else torch.full_like(C0, float("nan"))
        l0 = pgb.launch_count()
        pgb.gemm(1.5, A, B, beta, Cm)
        sync_ok()
        return Cm.cpu().numpy(), pgb.launch_count() - l0

    got, launches = run()
    assert pgb.last_path() == pgb.PATH_DMMA and launches == 2
    ref = pbo.gemm(1.5, beta, hC.copy(), hA, hB)
    assert normwise(got, ref) <= 1e-12
    assert backward_gemm(got, ref, 1.5, beta, hA, hB, hC) <= 1e-13
    again, _ = run()
    assert np.array_equal(got, again)
    pgb.init(no_split_k=1)   # split-K off
    try:
        unsplit, launches = run()
    finally:
        pgb.init()
    assert launches == 1 and normwise(got, unsplit) <= 1e-13


def test_dgemm_empty_and_k0():
    A = torch.zeros((4, 0), dtype=torch.float64, device=DEV)
    B = torch.zeros((0, 8), dtype=torch.float64, device=DEV)
    Cm = dev_fill(4, 8, torch.float64, 1, -1.0, 1.0)
    C0 = Cm.clone()
    pgb.gemm(1.5, A, B, 1.2, Cm)  # K == 0: C *= beta
    sync_ok()
    assert torch.equal(Cm, C0 * 1.2)
    lib = pgb.load()
    assert lib.pgb200Dgemm(None, 0, 8, 4, 1.0, None, 4, None, 8, 0.0, None, 8) == pgb.OK
    assert lib.pgb200Dgemm(None, 4, 8, 4, 1.0, Cm.data_ptr(), 2, Cm.data_ptr(), 8, 0.0,
                           Cm.data_ptr(), 8) == pgb.ERR_INVALID  # lda < K
    assert lib.pgb200Dgemm(None, -1, 8, 4, 1.0, None, 4, None, 8, 0.0, None, 8) == pgb.ERR_INVALID


def test_dgemm_full_size_rows_and_freivalds():
    """configs[1]: M=N=K=4096, inputs uniform [-1,1).  Oracle on a pseudo-random
    row subset (rows are independent in the loop nest) plus a Freivalds check of
    the whole product."""
    n = 4096
    A = dev_fill(n, n, torch.float64, 1, -1.0, 1.0)
    B = dev_fill(n, n, torch.float64, 2, -1.0, 1.0)
    Cm = dev_fill(n, n, torch.float64, 3, -1.0, 1.0)
    C0 = Cm.clone()
    pgb.gemm(1.5, A, B, 1.2, Cm)
    sync_ok()
    assert pgb.last_path() == pgb.PATH_DMMA
    rows = np.sort(np.random.default_rng(SEED).choice(n, 24, replace=False))
    rows = np.unique(np.concatenate([rows, [0, 127, 128, n - 1]]))
    hB = pbo.fill(n, n, np.float64, SEED, 2, -1.0, 1.0)
    for r in rows:
        hA = pbo.fill(1, n, np.float64, SEED, 1, -1.0, 1.0, row0=int(r))
        hC = pbo.fill(1, n, np.float64, SEED, 3, -1.0, 1.0, row0=int(r))
        ref = pbo.gemm(1.5, 1.2, hC, hA, hB)
        got = Cm[int(r)].cpu().numpy()[None, :]
        assert normwise(got, ref) <= 1e-12
    v = dev_fill(n, 1, torch.float64, 9, -1.0, 1.0)
    lhs = Cm @ v
    rhs = 1.5 * (A @ (B @ v)) + 1.2 * (C0 @ v)
    assert float((lhs - rhs).abs().max() / rhs.abs().max()) <= 1e-12


# --------------------------------------------------------------------------- 2mm
def test_chained_gemm_matches_2mm_oracle():
    ni, nj, nk, nl = 192, 160, 224, 256
    A = dev_fill(ni, nk, torch.float64, 1, -1.0, 1.0)
    B = dev_fill(nk, nj, torch.float64, 2, -1.0, 1.0)
    Cc = dev_fill(nj, nl, torch.float64, 3, -1.0, 1.0)
    D = dev_fill(ni, nl, torch.float64, 4, -1.0, 1.0)
    hA, hB, hC, hD = (t.cpu().numpy() for t in (A, B, Cc, D))
    tmp = torch.full((ni, nj), float("nan"), dtype=torch.float64, device=DEV)
    pgb.gemm(1.5, A, B, 0.0, tmp)       # nest 1: tmp = alpha*A*B
    pgb.gemm(1.0, tmp, Cc, 1.2, D)      # nest 2: D = tmp*C + beta*D
    sync_ok()
    htmp = np.zeros((ni, nj))
    ref = pbo.mm2(1.5, 1.2, htmp, hA, hB, hC, hD.copy())
    assert normwise(tmp.cpu().numpy(), htmp) <= 1e-12
    assert normwise(D.cpu().numpy(), ref) <= 1e-12


def test_dgemm_generic_kernels_still_selectable():
    """force_generic keeps the plain SIMT kernels reachable (any shape, no TMA)."""
    A = dev_fill(97, 45, torch.float64, 1, -1.0, 1.0)
    B = dev_fill(45, 61, torch.float64, 2, -1.0, 1.0)
    Cm = dev_fill(97, 61, torch.float64, 3, -1.0, 1.0)
    ref = pbo.gemm(1.5, 1.2, Cm.cpu().numpy(), A.cpu().numpy(), B.cpu().numpy())
    pgb.init(force_generic=1)
    try:
        pgb.gemm(1.5, A, B, 1.2, Cm)
        sync_ok()
        assert pgb.last_path() == pgb.PATH_SIMT
    finally:
        pgb.init()
    assert normwise(Cm.cpu().numpy(), ref) <= 1e-12


def test_dsyrk_odd_shapes_take_the_tensor_path():
    n, k = 45, 33
    A = dev_fill(n, k, torch.float64, 1, -1.0, 1.0)
    Cm = dev_fill(n, n, torch.float64, 2, -1.0, 1.0)
    hA, hC = np.ascontiguousarray(A.cpu().numpy()), np.ascontiguousarray(Cm.cpu().numpy())
    pgb.syrk(1.5, A, 1.2, Cm)
    sync_ok()
    assert pgb.last_path() == pgb.PATH_DMMA
    ref = pbo.syrk(1.5, 1.2, hC.copy(), hA)
    il = np.tril_indices(n)
    assert normwise(Cm.cpu().numpy()[il], ref[il]) <= 1e-12
    assert np.array_equal(Cm.cpu().numpy()[np.triu_indices(n, 1)], hC[np.triu_indices(n, 1)])


def test_chained_gemm_config3_full_size():
    """configs[3]: tmp = alpha*A*B, D = tmp*C + beta*D with A 4096x6144, B 6144x5120,
    C 5120x8192, D 4096x8192, inputs uniform [-1,1), alpha = 1.5, beta = 1.2.  Two
    calls on one stream with `tmp` NaN-filled first (beta == 0 must not read
    it); the loop nests on a row subset (rows of both nests are independent),
    Freivalds identities over all of tmp and D, and the host-array drop-in
    pgb200_kernel_2mm against the device-resident result."""
    ni, nk, nj, nl = 4096, 6144, 5120, 8192
    A = dev_fill(ni, nk, torch.float64, 1, -1.0, 1.0)
    B = dev_fill(nk, nj, torch.float64, 2, -1.0, 1.0)
    Cc = dev_fill(nj, nl, torch.float64, 3, -1.0, 1.0)
    D = dev_fill(ni, nl, torch.float64, 4, -1.0, 1.0)
    D0 = D.clone()
    tmp = torch.full((ni, nj), float("nan"), dtype=torch.float64, device=DEV)
    pgb.gemm(1.5, A, B, 0.0, tmp)
    pgb.gemm(1.0, tmp, Cc, 1.2, D)
    sync_ok()
    assert pgb.last_path() == pgb.PATH_DMMA
    assert not bool(torch.isnan(tmp).any()) and not bool(torch.isnan(D).any())
    # Freivalds: tmp v = alpha A (B v); D v = tmp (C v) + beta D0 v
    v1 = dev_fill(nj, 1, torch.float64, 9, -1.0, 1.0)
    lhs, rhs = tmp @ v1, 1.5 * (A @ (B @ v1))
    assert float((lhs - rhs).abs().max() / rhs.abs().max()) <= 1e-12
    v2 = dev_fill(nl, 1, torch.float64, 10, -1.0, 1.0)
    lhs, rhs = D @ v2, tmp @ (Cc @ v2) + 1.2 * (D0 @ v2)
    assert float((lhs - rhs).abs().max() / rhs.abs().max()) <= 1e-12
    # the nests themselves on a few rows (first/last row of a tile, first/last row)
    hB = pbo.fill(nk, nj, np.float64, SEED, 2, -1.0, 1.0)
    hC = pbo.fill(nj, nl, np.float64, SEED, 3, -1.0, 1.0)
    rows = [0, 127, 128, 2049, ni - 1]
    for r in rows:
        hA = pbo.fill(1, nk, np.float64, SEED, 1, -1.0, 1.0, row0=r)
        hD = pbo.fill(1, nl, np.float64, SEED, 4, -1.0, 1.0, row0=r)
        htmp = np.zeros((1, nj))
        ref = pbo.mm2(1.5, 1.2, htmp, hA, hB, hC, hD)
        assert normwise(tmp[r].cpu().numpy()[None, :], htmp) <= 1e-12
        assert normwise(D[r].cpu().numpy()[None, :], ref) <= 1e-12
    # the reference-named drop-in on host arrays gives the same arrays
    hA = pbo.fill(ni, nk, np.float64, SEED, 1, -1.0, 1.0)
    hD = pbo.fill(ni, nl, np.float64, SEED, 4, -1.0, 1.0)
    htmp = np.full((ni, nj), np.nan)
    polybench.kernel_2mm(ni, nj, nk, nl, 1.5, 1.2, htmp, hA, hB, hC, hD)
    assert np.array_equal(htmp, tmp.cpu().numpy())
    assert np.array_equal(hD, D.cpu().numpy())


# --------------------------------------------------------------------------- mat-vec
@pytest.mark.parametrize("n,pad", [(1, 0), (2, 0), (7, 0), (40, 0), (129, 0), (256, 0), (258, 6),
                                    (1000, 0), (1537, 3), (4096, 0)])
def test_mvt_matches_oracle(n, pad):
    A = dev_fill(n, n, torch.float64, 1, 0.0, 1.0, ld=n + pad)
    vec = [dev_fill(1, n, torch.float64, 2 + k, 0.0, 1.0).reshape(n).contiguous() for k in range(4)]
    x1, x2, y1, y2 = vec
    h = [t.cpu().numpy().copy() for t in vec]
    hA = np.ascontiguousarray(A.cpu().numpy())
    pgb.mvt(A, y1, y2, x1, x2)
    sync_ok()
    assert pgb.last_path() == pgb.PATH_STREAM
    pbo.mvt(h[0], h[1], h[2], h[3], hA)
    assert elementwise_rel(x1.cpu().numpy(), h[0]) <= 1e-12
    assert elementwise_rel(x2.cpu().numpy(), h[1]) <= 1e-12


@pytest.mark.parametrize("M,N", [(300, 200), (64, 1025), (1, 9), (513, 2)])
@pytest.mark.parametrize("trans", [0, 1])
def test_dgemv_matches_numpy(M, N, trans):
    A = dev_fill(M, N, torch.float64, 1, -1.0, 1.0)
    x = dev_fill(1, M if trans else N, torch.float64, 2, -1.0, 1.0).reshape(-1).contiguous()
    y = dev_fill(1, N if trans else M, torch.float64, 3, -1.0, 1.0).reshape(-1).contiguous()
    hA, hx, hy = A.cpu().numpy(), x.cpu().numpy(), y.cpu().numpy()
    pgb.gemv(trans, 1.5, A, x, 1.2, y)
    sync_ok()
    ref = 1.5 * ((hA.T if trans else hA) @ hx) + 1.2 * hy
    assert normwise(y.cpu().numpy(), ref) <= 1e-12
    y.fill_(float("nan"))
    pgb.gemv(trans, 1.0, A, x, 0.0, y)  # beta == 0 must not read y
    sync_ok()
    assert normwise(y.cpu().numpy(), (hA.T if trans else hA) @ hx) <= 1e-12


def test_mvt_large_row_subset():
    n = 8192
    A = dev_fill(n, n, torch.float64, 1, 0.0, 1.0)
    vec = [dev_fill(1, n, torch.float64, 2 + k, 0.0, 1.0).reshape(n).contiguous() for k in range(4)]
    x1, x2, y1, y2 = vec
    h = [t.cpu().numpy().copy() for t in vec]
    x1_before = x1.clone()
    pgb.mvt(A, y1, y2, x1, x2)
    sync_ok()
    hA = pbo.fill(n, n, np.float64, SEED, 1, 0.0, 1.0)
    pbo.mvt(h[0], h[1], h[2], h[3], hA, 1000, 1064)
    assert elementwise_rel(x1.cpu().numpy()[1000:1064], h[0][1000:1064]) <= 1e-12
    assert elementwise_rel(x2.cpu().numpy()[1000:1064], h[1][1000:1064]) <= 1e-12
    # whole-vector property: 1^T(A y1) == (A^T 1)^T y1
    ones = torch.ones(n, dtype=torch.float64, device=DEV)
    lhs = float((x1 - x1_before).sum())
    rhs = float(((A.T @ ones) * y1).sum())
    assert abs(lhs - rhs) <= 1e-11 * abs(rhs)


def test_mvt_config2_full_size():
    """configs[2]: x1 += A*y1, x2 += A^T*y2 at N = 32768 (A is 8 GiB, element offsets reach
    2^30 and byte offsets 2^33), inputs uniform [0,1).  The
    two nests on 70 scattered indices (x1[i] needs row i of A, x2[i] column i,
    regenerated on the host by the counter-based generator) and the adjoint
    identities over the whole vectors."""
    n = 32768
    A = dev_fill(n, n, torch.float64, 1, 0.0, 1.0)
    vec = [dev_fill(1, n, torch.float64, 2 + k, 0.0, 1.0).reshape(n).contiguous() for k in range(4)]
    x1, x2, y1, y2 = vec
    h = [t.cpu().numpy().copy() for t in vec]
    x1_0, x2_0 = x1.clone(), x2.clone()
    pgb.mvt(A, y1, y2, x1, x2)
    sync_ok()
    assert pgb.last_path() == pgb.PATH_STREAM
    ones = torch.ones(n, dtype=torch.float64, device=DEV)
    # 1^T (A y1) == (A^T 1)^T y1   and   1^T (A^T y2) == (A 1)^T y2
    lhs, rhs = float((x1 - x1_0).sum()), float(((A.T @ ones) * y1).sum())
    assert abs(lhs - rhs) <= 1e-11 * abs(rhs)
    lhs, rhs = float((x2 - x2_0).sum()), float(((A @ ones) * y2).sum())
    assert abs(lhs - rhs) <= 1e-11 * abs(rhs)
    g1, g2 = x1.cpu().numpy(), x2.cpu().numpy()
    del A, ones
    torch.cuda.empty_cache()
    hA = pbo.fill(n, n, np.float64, SEED, 1, 0.0, 1.0)
    idx = np.random.default_rng(SEED).choice(n, 62, replace=False)
    idx = np.unique(np.concatenate([idx, [0, 1, 255, 256, 257, n // 2, n - 2, n - 1]]))
    assert len(idx) >= 64
    r1, r2 = h[0].copy(), h[1].copy()
    for i in idx:
        pbo.mvt(r1, r2, h[2], h[3], hA, int(i), int(i) + 1)
    assert elementwise_rel(g1[idx], r1[idx]) <= 1e-12
    assert elementwise_rel(g2[idx], r2[idx]) <= 1e-12
    # every other entry changed too (x += positive sums)
    assert np.all(g1 > h[0]) and np.all(g2 > h[1])


# --------------------------------------------------------------------------- syrk
@pytest.mark.parametrize("n,k,pa,pc", [(128, 64, 0, 0), (300, 100, 0, 0), (257, 36, 2, 4),
                                        (45, 33, 0, 0), (1, 4, 0, 0),
                                        (384, 1024, 0, 0), (1200, 1000, 0, 0)])  # split-K
def test_dsyrk_matches_oracle(n, k, pa, pc):
    A = dev_fill(n, k, torch.float64, 1, -1.0, 1.0, ld=k + pa)
    Cm = dev_fill(n, n, torch.float64, 2, -1.0, 1.0, ld=n + pc)
    hA, hC = np.ascontiguousarray(A.cpu().numpy()), np.ascontiguousarray(Cm.cpu().numpy())
    C0 = hC.copy()
    pgb.syrk(1.5, A, 1.2, Cm)
    sync_ok()
    ref = pbo.syrk(1.5, 1.2, hC, hA)
    got = Cm.cpu().numpy()
    il = np.tril_indices(n)
    assert normwise(got[il], ref[il]) <= 1e-12
    iu = np.triu_indices(n, 1)
    assert np.array_equal(got[iu], C0[iu]), "strict upper triangle must stay untouched"


# --------------------------------------------------------------------------- fp32 (path-agnostic gates)
def _sgemm_case(M, N, K, beta=1.2):
    A = dev_fill(M, K, torch.float32, 1, 0.0, 1.0)
    B = dev_fill(K, N, torch.float32, 2, 0.0, 1.0)
    Cm = dev_fill(M, N, torch.float32, 3, 0.0, 1.0)
    hA, hB, hC = (np.ascontiguousarray(t.cpu().numpy()) for t in (A, B, Cm))
    pgb.gemm(1.5, A, B, beta, Cm)
    sync_ok()
    got = Cm.cpu().numpy()
    truth = pbo.gemm_acc64(1.5, beta, hC, hA, hB)
    seq = pbo.gemm(1.5, beta, hC.copy(), hA, hB)
    return got, truth, seq


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 1024), (200, 136, 100), (97, 61, 45),
                                    (1, 4, 4), (384, 256, 4096)])
def test_sgemm_matches_oracle(M, N, K):
    got, truth, seq = _sgemm_case(M, N, K)
    assert elementwise_rel(got, truth) <= 1e-5
    assert elementwise_rel(got, seq) <= 1e-5


@pytest.mark.parametrize("M,N,K,beta", [(512, 512, 2048, 1.2), (256, 384, 1000, 0.0),
                                         (1000, 1100, 1200, 1.2), (130, 250, 4100, 1.2)])
def test_sgemm_split_k(M, N, K, beta):
    """Few tiles, long K: the K-blocks of each tile are dealt to several CTAs and
    the partial products are added in a fixed order.  Operands that can be used
    in place take the fused kernel (one launch: lo parts made in shared memory,
    K split inside a cluster, partial tiles added over distributed shared
    memory); the others take split, product and reduce (3 or 4 launches).
    Ragged edges in all three extents; beta == 0 must not read C; two runs give
    the same bits; the result agrees with the unsplit kernel."""
    l0 = pgb.launch_count()
    got, truth, seq = _sgemm_case(M, N, K, beta)
    fused = (K % 4 == 0) and (N % 4 == 0)      # 16-byte aligned rows of A and B
    # 3 input fills, then: the fused kernel | operand planes (one launch, two when
    # B has to be transposed) + split-K product + reduce
    assert pgb.launch_count() - l0 == (4 if fused else 7)
    assert pgb.last_path() == pgb.PATH_TCGEN05
    assert elementwise_rel(got, truth) <= 1e-5
    if K <= 2048:
        assert elementwise_rel(got, seq) <= 1e-5
    again, _, _ = _sgemm_case(M, N, K, beta)
    assert np.array_equal(got, again)
    if beta == 0.0:
        A = dev_fill(M, K, torch.float32, 1, 0.0, 1.0)
        B = dev_fill(K, N, torch.float32, 2, 0.0, 1.0)
        Cn = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
        pgb.gemm(1.5, A, B, 0.0, Cn)
        sync_ok()
        assert np.array_equal(Cn.cpu().numpy(), got)
    pgb.init(no_split_k=1)   # split-K off
    try:
        unsplit, _, _ = _sgemm_case(M, N, K, beta)
    finally:
        pgb.init()
    assert elementwise_rel(got, unsplit) <= 1e-5


@pytest.mark.parametrize("M,N,K", [(2560, 2304, 2048), (2048, 2832, 2048)])
def test_sgemm_round_meeting_changes_no_bit(M, N, K):
    """More tiles than CTAs and K >= 2048: the TMA producers of the persistent
    fp32 kernels meet between rounds of tiles so that CTAs sharing an operand
    panel stay close in K (two-CTA kernel: 10 x 9 pair tiles on 74 pairs;
    one-CTA kernel, N % 32 != 0: 16 x 12 tiles on 148 CTAs).  The meeting only
    changes when loads are issued: the bits are those of a run with
    pgb200Config.no_step_sync, also when two such products run at once on two
    streams (the CTAs of the second grid cannot all be running, so its
    producers give the meeting up), and they match the fp64-accumulated product."""
    A = dev_fill(M, K, torch.float32, 1, 0.0, 1.0)
    B = dev_fill(K, N, torch.float32, 2, 0.0, 1.0)
    C0 = dev_fill(M, N, torch.float32, 3, 0.0, 1.0)

    def run():
        Cm = C0.clone()
        pgb.gemm(1.5, A, B, 1.2, Cm)
        sync_ok()
        return Cm

    met = run()
    assert pgb.last_path() == pgb.PATH_TCGEN05
    pgb.init(no_step_sync=1)
    try:
        alone = run()
    finally:
        pgb.init()
    assert torch.equal(met, alone)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    C1, C2 = C0.clone(), C0.clone()
    torch.cuda.synchronize()
    with torch.cuda.stream(s1):
        pgb.gemm(1.5, A, B, 1.2, C1)
    with torch.cuda.stream(s2):
        pgb.gemm(1.5, A, B, 1.2, C2)
    sync_ok()
    assert torch.equal(C1, met) and torch.equal(C2, met)
    hA, hB, hC = (t.cpu().numpy().astype(np.float64) for t in (A, B, C0))
    truth = 1.5 * (hA @ hB) + 1.2 * hC
    assert elementwise_rel(met.cpu().numpy(), truth) <= 1e-5


@pytest.mark.parametrize("M,N,K,beta", [(200, 300, 400, 1.0), (100, 300, 200, 0.0)])
def test_sgemm_plain_matmul_nests(M, N, K, beta):
    """The two fp32 matmul nests of the reference's raise-to-affine test
    (tools/cgeist/Test/Verification/raiseToAffine.c:12-27 `C += A*B`, and :30-51
    `C = 0; C += A*B`), through the drop-in with alpha = 1 and beta = 1 / 0."""
    A = pbo.fill(M, K, np.float32, SEED, 1, 0.0, 1.0)
    B = pbo.fill(K, N, np.float32, SEED, 2, 0.0, 1.0)
    C0 = pbo.fill(M, N, np.float32, SEED, 3, 0.0, 1.0)
    got = C0.copy() if beta else np.full((M, N), np.nan, dtype=np.float32)
    polybench.kernel_gemm(M, N, K, 1.0, beta, got, A, B)
    # the nest itself, sequential fp32 (alpha = 1 and beta = 1 are exact factors)
    seq = pbo.gemm(1.0, beta, C0.copy() if beta else np.zeros((M, N), np.float32), A, B)
    truth = pbo.gemm_acc64(1.0, beta, C0, A, B)
    assert elementwise_rel(got, truth) <= 1e-5
    assert elementwise_rel(got, seq) <= 1e-5


def test_sgemm_config0_1024():
    """configs[0]: fp32 M=N=K=1024, uniform [0,1), alpha=1.5, beta=1.2."""
    l0 = pgb.launch_count()
    got, truth, seq = _sgemm_case(1024, 1024, 1024)
    assert pgb.launch_count() - l0 == 4        # 3 input fills + ONE kernel for the product
    assert elementwise_rel(got, truth) <= 1e-5
    assert elementwise_rel(got, seq) <= 1e-5
    again, _, _ = _sgemm_case(1024, 1024, 1024)
    assert np.array_equal(got, again)


@pytest.mark.parametrize("n,k", [(128, 64), (300, 100), (45, 33), (512, 1024), (1200, 1000)])
def test_ssyrk_matches_oracle(n, k):
    A = dev_fill(n, k, torch.float32, 1, 0.0, 1.0)
    Cm = dev_fill(n, n, torch.float32, 2, 0.0, 1.0)
    hA, hC = np.ascontiguousarray(A.cpu().numpy()), np.ascontiguousarray(Cm.cpu().numpy())
    C0 = hC.copy()
    pgb.syrk(1.5, A, 1.2, Cm)
    sync_ok()
    got = Cm.cpu().numpy()
    truth = pbo.syrk_acc64(1.5, 1.2, hC, hA)
    seq = pbo.syrk(1.5, 1.2, hC.copy(), hA)
    il = np.tril_indices(n)
    assert elementwise_rel(got[il], truth[il]) <= 1e-5
    assert elementwise_rel(got[il], seq[il]) <= 1e-5
    iu = np.triu_indices(n, 1)
    assert np.array_equal(got[iu], C0[iu])


@pytest.mark.parametrize("n,k,blocks", [
    (384, 128, [(0, 100), (100, 256), (256, 384)]),            # one-CTA kernel, 128x64 tiles
    (2048, 256, [(0, 640), (640, 1408), (1408, 2048)]),        # two-CTA kernel, row0 != 0
    (640, 1024, [(0, 200), (200, 640)]),                       # split-K with row0 != 0, ragged block
])
def test_ssyrk_row_block_equals_rows_of_full_update(n, k, blocks):
    A = dev_fill(n, k, torch.float32, 1, 0.0, 1.0)
    C1 = dev_fill(n, n, torch.float32, 2, 0.0, 1.0)
    C2 = C1.clone()
    C0 = C1.clone()
    pgb.syrk(1.5, A, 1.2, C1)
    for r0, r1 in blocks:
        pgb.syrk(1.5, A, 1.2, C2, rows=(r0, r1))
    sync_ok()
    il = np.tril_indices(n)
    assert elementwise_rel(C2.cpu().numpy()[il], C1.cpu().numpy()[il]) <= 1e-6
    truth = 1.5 * (A.double() @ A.double().T) + 1.2 * C0.double()
    assert elementwise_rel(C1.cpu().numpy()[il], truth.cpu().numpy()[il]) <= 1e-5
    iu = np.triu_indices(n, 1)
    assert np.array_equal(C2.cpu().numpy()[iu], C0.cpu().numpy()[iu])


def test_ssyrk_config4_full_size():
    """configs[4]a: fp32 SYRK N=16384, K=8192, inputs uniform [0,1).  CPU oracle on
    scattered rows; every lower-triangle entry against an fp64 evaluation on the
    GPU; strict upper triangle untouched."""
    n, k = 16384, 8192
    A = dev_fill(n, k, torch.float32, 1, 0.0, 1.0)
    Cm = dev_fill(n, n, torch.float32, 2, 0.0, 1.0)
    C0 = Cm.clone()
    pgb.syrk(1.5, A, 1.2, Cm)
    sync_ok()
    assert pgb.last_path() == pgb.PATH_TCGEN05
    hA = pbo.fill(n, k, np.float32, SEED, 1, 0.0, 1.0)
    for r in (0, 127, 128, 255, 256, 5000, 11111, n - 1):
        hC = pbo.fill(1, n, np.float32, SEED, 2, 0.0, 1.0, row0=r)
        truth = pbo.syrk_block(1.5, 1.2, hC, hA, r, acc64=True)[0, : r + 1]
        seq = pbo.syrk_block(1.5, 1.2, hC.copy(), hA, r)[0, : r + 1]
        got = Cm[r, : r + 1].cpu().numpy()
        assert elementwise_rel(got, truth) <= 1e-5
        assert elementwise_rel(got, seq) <= 1e-5
    Ad = A.double()
    worst = 0.0
    for r0 in range(0, n, 2048):
        t = 1.5 * (Ad[r0:r0 + 2048] @ Ad.T) + 1.2 * C0[r0:r0 + 2048].double()
        g = Cm[r0:r0 + 2048].double()
        rows = torch.arange(r0, r0 + 2048, device=DEV)[:, None]
        cols = torch.arange(n, device=DEV)[None, :]
        low = cols <= rows
        worst = max(worst, float((((g - t).abs() / t.abs())[low]).max()))
        assert torch.equal(Cm[r0:r0 + 2048][~low], C0[r0:r0 + 2048][~low])
    assert worst <= 1e-5


def test_sgemm_config4_full_size():
    """configs[4]b: fp32 GEMM M=N=K=32768, inputs uniform [0,1).  K exceeds 8192, so
    the gate is the fp64-accumulated evaluation of the same fp32 inputs (the
    sequential fp32 nest is itself ~1e-5 from it at this K): CPU oracle on two
    rows, GPU fp64 on 128 pseudo-random rows plus block-boundary rows, and a
    Freivalds identity over the whole product."""
    n = 32768
    A = dev_fill(n, n, torch.float32, 1, 0.0, 1.0)
    B = dev_fill(n, n, torch.float32, 2, 0.0, 1.0)
    Cm = dev_fill(n, n, torch.float32, 3, 0.0, 1.0)
    C0 = Cm.clone()
    pgb.gemm(1.5, A, B, 1.2, Cm)
    sync_ok()
    assert pgb.last_path() == pgb.PATH_TCGEN05
    rows = np.random.default_rng(SEED).choice(n, 128, replace=False)
    rows = np.unique(np.concatenate([rows, [0, 127, 128, 4095, 4096, n // 2 - 1, n // 2, n - 1]]))
    idx = torch.from_numpy(rows).to(DEV)
    Bd = B.double()
    truth = 1.5 * (A[idx].double() @ Bd) + 1.2 * C0[idx].double()
    got = Cm[idx].double()
    assert float(((got - truth).abs() / truth.abs()).max()) <= 1e-5
    v = dev_fill(n, 1, torch.float64, 9, 0.0, 1.0)
    lhs = Cm.double() @ v
    rhs = 1.5 * (A.double() @ (Bd @ v)) + 1.2 * (C0.double() @ v)
    assert float(((lhs - rhs).abs() / rhs.abs()).max()) <= 1e-5
    del Bd, lhs, rhs, truth, got
    hB = pbo.fill(n, n, np.float32, SEED, 2, 0.0, 1.0)
    for r in (1, n - 2):
        hA = pbo.fill(1, n, np.float32, SEED, 1, 0.0, 1.0, row0=r)
        hC = pbo.fill(1, n, np.float32, SEED, 3, 0.0, 1.0, row0=r)
        t = pbo.gemm_acc64(1.5, 1.2, hC, hA, hB)
        assert elementwise_rel(Cm[r].cpu().numpy()[None, :], t) <= 1e-5


# --------------------------------------------------------------------------- reference-style drop-ins (host arrays)
@pytest.mark.parametrize("tname,dtype", [("f64", np.float64), ("f32", np.float32)])
def test_kernel_gemm_dropin_reproduces_golden_dump(tname, dtype):
    ni, nj, nk = MINI["gemm"]
    alpha, beta, Cm, A, B = init_gemm(ni, nj, nk, dtype)
    polybench.kernel_gemm(ni, nj, nk, alpha, beta, Cm, A, B)
    assert_dump_equal(read_dump("gemm", tname)["C"], Cm, slack_ulps=1)


def test_kernel_2mm_dropin_reproduces_golden_dump():
    ni, nj, nk, nl = MINI["2mm"]
    alpha, beta, tmp, A, B, Cm, D = init_2mm(ni, nj, nk, nl, np.float64)
    polybench.kernel_2mm(ni, nj, nk, nl, alpha, beta, tmp, A, B, Cm, D)
    assert_dump_equal(read_dump("2mm", "f64")["D"], D, slack_ulps=1)
    assert normwise(tmp, 1.5 * (A @ B)) <= 1e-12


def test_kernel_mvt_dropin_reproduces_golden_dump():
    (n,) = MINI["mvt"]
    x1, x2, y1, y2, A = init_mvt(n, np.float64)
    polybench.kernel_mvt(n, x1, x2, y1, y2, A)
    d = read_dump("mvt", "f64")
    assert_dump_equal(d["x1"], x1, slack_ulps=1)
    assert_dump_equal(d["x2"], x2, slack_ulps=1)


@pytest.mark.parametrize("tname,dtype", [("f64", np.float64), ("f32", np.float32)])
def test_kernel_syrk_dropin_reproduces_golden_dump(tname, dtype):
    n, m = MINI["syrk"]
    alpha, beta, Cm, A = init_syrk(n, m, dtype)
    polybench.kernel_syrk(n, m, alpha, beta, Cm, A)
    assert_dump_equal(read_dump("syrk", tname)["C"], Cm, slack_ulps=1)


@pytest.mark.parametrize("M,N", [(300, 200), (42, 38), (1030, 517), (2048, 4096)])
def test_gemv_pair_matches_bicg_oracle(M, N):
    """bicg nest: A is M x N (PolyBench's n x m), q = A p, s = A^T r, one pass."""
    A = dev_fill(M, N, torch.float64, 1, 0.0, 1.0)
    p = dev_fill(1, N, torch.float64, 2, 0.0, 1.0).reshape(N).contiguous()
    r = dev_fill(1, M, torch.float64, 3, 0.0, 1.0).reshape(M).contiguous()
    q = torch.full((M,), float("nan"), dtype=torch.float64, device=DEV)
    s = torch.full((N,), float("nan"), dtype=torch.float64, device=DEV)
    pgb.gemv_pair(1.0, A, p, r, 0.0, q, s)
    sync_ok()
    hs, hq = np.zeros(N), np.zeros(M)
    pbo.bicg(np.ascontiguousarray(A.cpu().numpy()), hs, hq, p.cpu().numpy(), r.cpu().numpy())
    assert elementwise_rel(q.cpu().numpy(), hq) <= 1e-12
    assert elementwise_rel(s.cpu().numpy(), hs) <= 1e-12


def test_same_shaped_nests_reproduce_golden_dumps():
    """3mm / atax / bicg / gesummv drop-ins on the reference's MINI inputs."""
    ni, nj, nk, nl, nm = MINI["3mm"]
    E, A, B, F, Cm, D, G = init_3mm(ni, nj, nk, nl, nm, np.float64)
    polybench.kernel_3mm(ni, nj, nk, nl, nm, E, A, B, F, Cm, D, G)
    assert_dump_equal(read_dump("3mm", "f64")["G"], G, slack_ulps=1)
    assert normwise(E, A @ B) <= 1e-12 and normwise(F, Cm @ D) <= 1e-12
    m, n = MINI["atax"]
    A, x, y, tmp = init_atax(m, n, np.float64)
    polybench.kernel_atax(m, n, A, x, y, tmp)
    assert_dump_equal(read_dump("atax", "f64")["y"], y, slack_ulps=1)
    assert normwise(tmp, A @ x) <= 1e-12
    m, n = MINI["bicg"]
    A, s, q, p, r = init_bicg(m, n, np.float64)
    polybench.kernel_bicg(m, n, A, s, q, p, r)
    d = read_dump("bicg", "f64")
    assert_dump_equal(d["s"], s, slack_ulps=1)
    assert_dump_equal(d["q"], q, slack_ulps=1)
    (n,) = MINI["gesummv"]
    alpha, beta, A, B, tmp, x, y = init_gesummv(n, np.float64)
    polybench.kernel_gesummv(n, alpha, beta, A, B, tmp, x, y)
    assert_dump_equal(read_dump("gesummv", "f64")["y"], y, slack_ulps=1)


def test_same_shaped_nests_match_oracle_on_seeded_inputs():
    ni, nj, nk, nl, nm = 160, 136, 200, 184, 96
    h = [pbo.fill(r, c, np.float64, SEED, k, -1.0, 1.0) for k, (r, c) in
         enumerate([(ni, nk), (nk, nj), (nj, nm), (nm, nl)], 1)]
    E, F, G = np.zeros((ni, nj)), np.zeros((nj, nl)), np.zeros((ni, nl))
    E2, F2, G2 = E.copy(), F.copy(), G.copy()
    polybench.kernel_3mm(ni, nj, nk, nl, nm, E, h[0], h[1], F, h[2], h[3], G)
    pbo.mm3(E2, h[0], h[1], F2, h[2], h[3], G2)
    assert normwise(G, G2) <= 1e-12 and normwise(E, E2) <= 1e-12 and normwise(F, F2) <= 1e-12
    m, n = 700, 500
    A = pbo.fill(m, n, np.float64, SEED, 5, 0.0, 1.0)
    x = pbo.fill_vec(n, np.float64, SEED, 6, 0.0, 1.0)
    y, tmp, y2, tmp2 = np.zeros(n), np.zeros(m), np.zeros(n), np.zeros(m)
    polybench.kernel_atax(m, n, A, x, y, tmp)
    pbo.atax(A, x, y2, tmp2)
    assert elementwise_rel(y, y2) <= 1e-12 and elementwise_rel(tmp, tmp2) <= 1e-12
    n = 600
    A = pbo.fill(n, n, np.float64, SEED, 7, 0.0, 1.0)
    B = pbo.fill(n, n, np.float64, SEED, 8, 0.0, 1.0)
    x = pbo.fill_vec(n, np.float64, SEED, 9, 0.0, 1.0)
    y, tmp, y2, tmp2 = np.zeros(n), np.zeros(n), np.zeros(n), np.zeros(n)
    polybench.kernel_gesummv(n, 1.5, 1.2, A, B, tmp, x, y)
    pbo.gesummv(1.5, 1.2, A, B, tmp2, x, y2)
    assert elementwise_rel(y, y2) <= 1e-12 and elementwise_rel(tmp, tmp2) <= 1e-12


@pytest.mark.parametrize("dtype,np_dtype", [(torch.float64, np.float64), (torch.float32, np.float32)])
@pytest.mark.parametrize("M,N,K", [(256, 384, 128), (200, 136, 100), (97, 61, 45)])
def test_gemm_nt_matches_numpy(dtype, np_dtype, M, N, K):
    lo = -1.0 if dtype == torch.float64 else 0.0
    A = dev_fill(M, K, dtype, 1, lo, 1.0)
    B = dev_fill(N, K, dtype, 2, lo, 1.0)
    Cm = dev_fill(M, N, dtype, 3, lo, 1.0)
    truth = 1.5 * (A.double() @ B.double().T) + 1.2 * Cm.double()
    pgb.gemm_nt(1.5, A, B, 1.2, Cm)
    sync_ok()
    if dtype == torch.float64:
        assert float((Cm - truth).abs().max() / truth.abs().max()) <= 1e-12
    else:
        assert float(((Cm.double() - truth).abs() / truth.abs()).max()) <= 1e-5


@pytest.mark.parametrize("np_dtype,tname", [(np.float64, "f64"), (np.float32, "f32")])
def test_syr2k_matches_oracle_and_golden(np_dtype, tname):
    n, m = MINI["syr2k"]
    alpha, beta, Cm, A, B = init_syr2k(n, m, np_dtype)
    polybench.kernel_syr2k(n, m, alpha, beta, Cm, A, B)
    assert_dump_equal(read_dump("syr2k", tname)["C"], Cm, slack_ulps=1)
    n, k = 300, 136
    A = pbo.fill(n, k, np_dtype, SEED, 1, 0.0, 1.0)
    B = pbo.fill(n, k, np_dtype, SEED, 2, 0.0, 1.0)
    C0 = pbo.fill(n, n, np_dtype, SEED, 3, 0.0, 1.0)
    got = C0.copy()
    polybench.kernel_syr2k(n, k, 1.5, 1.2, got, A, B)
    ref = pbo.syr2k(1.5, 1.2, C0.copy(), A, B)
    il, iu = np.tril_indices(n), np.triu_indices(n, 1)
    assert elementwise_rel(got[il], ref[il]) <= (1e-12 if np_dtype == np.float64 else 1e-5)
    assert np.array_equal(got[iu], C0[iu])


@pytest.mark.parametrize("np_dtype,tname", [(np.float64, "f64"), (np.float32, "f32")])
def test_symm_matches_oracle_and_golden(np_dtype, tname):
    m, n = MINI["symm"]
    alpha, beta, Cm, A, B = init_symm(m, n, np_dtype)   # upper triangle of A holds -999
    polybench.kernel_symm(m, n, alpha, beta, Cm, A, B)
    assert_dump_equal(read_dump("symm", tname)["C"], Cm, slack_ulps=1)
    tol = 1e-12 if np_dtype == np.float64 else 1e-5
    for m, n in ((300, 260), (512, 384), (1001, 128)):
        A = pbo.fill(m, m, np_dtype, SEED, 1, 0.0, 1.0)
        A[np.triu_indices(m, 1)] = np.nan               # must never be read
        B = pbo.fill(m, n, np_dtype, SEED, 2, 0.0, 1.0)
        C0 = pbo.fill(m, n, np_dtype, SEED, 3, 0.0, 1.0)
        got = C0.copy()
        polybench.kernel_symm(m, n, 1.5, 1.2, got, A, B)
        ref = pbo.symm(1.5, 1.2, C0.copy(), A, B)
        assert np.isfinite(got).all()
        assert elementwise_rel(got, ref) <= tol, (m, n)


@pytest.mark.parametrize("np_dtype,tname", [(np.float64, "f64"), (np.float32, "f32")])
def test_trmm_matches_oracle_and_golden(np_dtype, tname):
    m, n = MINI["trmm"]
    alpha, A, B = init_trmm(m, n, np_dtype)
    polybench.kernel_trmm(m, n, alpha, A, B)
    assert_dump_equal(read_dump("trmm", tname)["B"], B, slack_ulps=1)
    tol = 1e-12 if np_dtype == np.float64 else 1e-5
    # 1000 rows: four row blocks, inner extent padded; 515: odd extents everywhere
    for m, n in ((300, 260), (1000, 256), (515, 77), (2304, 128), (2304, 1280)):
        A = pbo.fill(m, m, np_dtype, SEED, 1, 0.0, 1.0)
        A[np.triu_indices(m, 0)] = np.nan               # diagonal and above: never read
        B0 = pbo.fill(m, n, np_dtype, SEED, 2, 0.0, 1.0)
        got = B0.copy()
        polybench.kernel_trmm(m, n, 1.5, A, got)
        ref = pbo.trmm(1.5, A, B0.copy())
        assert np.isfinite(got).all()
        assert elementwise_rel(got, ref) <= tol, (m, n)


def test_doitgen_matches_oracle_and_golden():
    nr, nq, np_ = MINI["doitgen"]
    A, C4, sum_ = init_doitgen(nr, nq, np_, np.float64)
    polybench.kernel_doitgen(nr, nq, np_, A, C4, sum_)
    assert_dump_equal(read_dump("doitgen", "f64")["A"], A, slack_ulps=1)
    assert np.array_equal(sum_, A[-1, -1])
    for nr, nq, np_ in ((20, 25, 128), (7, 9, 30), (50, 40, 160)):   # the last is PolyBench MEDIUM
        A = pbo.fill(nr * nq, np_, np.float64, SEED, 1, -1.0, 1.0).reshape(nr, nq, np_)
        C4 = pbo.fill(np_, np_, np.float64, SEED, 2, -1.0, 1.0)
        got, s1, s2 = A.copy(), np.zeros(np_), np.zeros(np_)
        polybench.kernel_doitgen(nr, nq, np_, got, C4, s1)
        ref = pbo.doitgen(A.copy(), C4, s2)
        assert normwise(got, ref) <= 1e-12
        assert np.array_equal(s1, got[-1, -1])


def test_symm_trmm_doitgen_device_pointers_on_a_stream():
    """Device-pointer forms, padded leading dimensions, non-default stream."""
    m, n = 640, 384
    st = torch.cuda.Stream(device=DEV)
    A = dev_fill(m, m, torch.float64, 1, 0.0, 1.0, ld=m + 4)
    B = dev_fill(m, n, torch.float64, 2, 0.0, 1.0, ld=n + 8)
    Cm = dev_fill(m, n, torch.float64, 3, 0.0, 1.0, ld=n + 2)
    hA, hB, hC = (t.cpu().numpy().copy() for t in (A, B, Cm))
    torch.cuda.synchronize()
    with torch.cuda.stream(st):
        pgb.symm(1.5, A, B, 1.2, Cm)
        assert pgb.last_path() == pgb.PATH_DMMA
        pgb.trmm(1.5, A, B)
    st.synchronize()
    sync_ok()
    assert elementwise_rel(Cm.cpu().numpy(), pbo.symm(1.5, 1.2, hC, hA, hB)) <= 1e-12
    assert elementwise_rel(B.cpu().numpy(), pbo.trmm(1.5, hA, hB.copy())) <= 1e-12
    r, p = 1500, 256
    A3 = dev_fill(r, p, torch.float64, 4, -1.0, 1.0)
    C4 = dev_fill(p, p, torch.float64, 5, -1.0, 1.0)
    h3, h4 = A3.cpu().numpy().copy(), C4.cpu().numpy().copy()
    s_dev = torch.zeros(p, dtype=torch.float64, device=DEV)
    pgb.doitgen(A3, C4, s_dev)
    sync_ok()
    ref = pbo.doitgen(h3, h4, np.zeros(p))
    assert normwise(A3.cpu().numpy(), ref) <= 1e-12
    assert torch.equal(s_dev, A3[-1])


def test_symm_trmm_doitgen_empty_and_rejected_arguments():
    lib = pgb.load()
    B = dev_fill(8, 6, torch.float64, 1, 0.0, 1.0)
    B0 = B.clone()
    p = B.data_ptr()
    # empty extents: nothing is touched, null pointers are fine
    assert lib.pgb200Dsymm(None, 0, 6, 1.5, None, 1, None, 6, 1.2, None, 6) == pgb.OK
    assert lib.pgb200Dtrmm(None, 8, 0, 1.5, None, 8, None, 1) == pgb.OK
    assert lib.pgb200Ddoitgen(None, 0, 6, None, 6, None, 6, None) == pgb.OK
    # negative sizes, null operands, leading dimensions below the row length
    assert lib.pgb200Dsymm(None, -1, 6, 1.5, p, 8, p, 6, 1.2, p, 6) == pgb.ERR_INVALID
    assert lib.pgb200Dsymm(None, 8, 6, 1.5, None, 8, p, 6, 1.2, p, 6) == pgb.ERR_INVALID
    assert lib.pgb200Dsymm(None, 8, 6, 1.5, p, 7, p, 6, 1.2, p, 6) == pgb.ERR_INVALID   # lda < M
    assert lib.pgb200Dtrmm(None, 8, 6, 1.5, p, 8, p, 5) == pgb.ERR_INVALID              # ldb < N
    assert lib.pgb200Strmm(None, 8, 6, 1.5, p, 8, None, 6) == pgb.ERR_INVALID
    assert lib.pgb200Ddoitgen(None, 8, 6, p, 5, p, 6, None) == pgb.ERR_INVALID          # lda < NP
    assert b"doitgen" in lib.pgb200GetLastErrorString()
    sync_ok()
    assert torch.equal(B, B0), "a rejected call must leave its arrays alone"
    # a 1x1 triangular factor is the identity: B = alpha * B
    A1 = torch.full((1, 1), float("nan"), dtype=torch.float64, device=DEV)
    row = dev_fill(1, 6, torch.float64, 2, 0.0, 1.0)
    r0 = row.clone()
    pgb.trmm(1.5, A1, row)
    sync_ok()
    assert torch.equal(row, r0 * 1.5)


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-12), (torch.float32, 1e-5)])
def test_symm_trmm_large_against_row_samples(dtype, tol):
    """4096-row operands: the triangular K loop runs over several rounds of
    tiles (DMMA kernel for fp64, two-CTA tcgen05 kernel for fp32).  Sampled
    rows are recomputed in float64 from the definition of each nest."""
    m, n = 4096, 2048
    A = dev_fill(m, m, dtype, 1, 0.0, 1.0)
    B = dev_fill(m, n, dtype, 2, 0.0, 1.0)
    Cm = dev_fill(m, n, dtype, 3, 0.0, 1.0)
    hA, hB, hC = (t.cpu().numpy().astype(np.float64) for t in (A, B, Cm))
    # poison what the nests never read
    iu = torch.triu_indices(m, m, 1, device=DEV)
    A_sym = A.clone()
    A_sym[iu[0], iu[1]] = float("nan")
    pgb.symm(1.5, A_sym, B, 1.2, Cm)
    A_tri = A_sym.clone()
    A_tri.fill_diagonal_(float("nan"))
    Bt = B.clone()
    pgb.trmm(1.5, A_tri, Bt)
    sync_ok()
    assert pgb.last_path() == (pgb.PATH_DMMA if dtype == torch.float64 else pgb.PATH_TCGEN05)
    rows = np.unique(np.concatenate([[0, 1, 127, 128, 255, 256, m - 129, m - 2, m - 1],
                                     np.random.default_rng(SEED).integers(0, m, 40)]))
    L = np.tril(hA)                                     # lower triangle, diagonal included
    gotC, gotB = Cm.cpu().numpy().astype(np.float64), Bt.cpu().numpy().astype(np.float64)
    assert np.isfinite(gotC).all() and np.isfinite(gotB).all()
    for i in rows:
        s_row = np.concatenate([L[i, : i + 1], L[i + 1:, i]])          # row i of the symmetric S
        ref_c = 1.2 * hC[i] + 1.5 * (s_row @ hB)
        assert elementwise_rel(gotC[i], ref_c) <= tol, ("symm", i)
        ref_b = 1.5 * (hB[i] + L[i + 1:, i] @ hB[i + 1:])
        assert elementwise_rel(gotB[i], ref_b) <= tol, ("trmm", i)


def test_plain_c_caller_runs_the_drop_ins(tmp_path):
    """The C ABI used from C: a PolyBench-style program calls the drop-ins on
    malloc'd arrays and checks them against its own loop nests."""
    import subprocess
    from test_abi import build_c_caller
    r = subprocess.run([build_c_caller(tmp_path), "--compute"], capture_output=True, text=True)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout + r.stderr


def test_gemver_matches_oracle_and_golden():
    (n,) = MINI["gemver"]
    alpha, beta, A, u1, v1, u2, v2, w, x, y, z = init_gemver(n, np.float64)
    polybench.kernel_gemver(n, alpha, beta, A, u1, v1, u2, v2, w, x, y, z)
    assert_dump_equal(read_dump("gemver", "f64")["w"], w, slack_ulps=1)
    for n in (700, 1030):
        A = pbo.fill(n, n, np.float64, SEED, 1, 0.0, 1.0)
        v = [pbo.fill_vec(n, np.float64, SEED, 2 + k, 0.0, 1.0) for k in range(8)]
        A2, v2_ = A.copy(), [t.copy() for t in v]
        polybench.kernel_gemver(n, 1.5, 1.2, A, *v)
        pbo.gemver(1.5, 1.2, A2, *v2_)
        assert np.array_equal(A, A2), "rank-2 update is rounded like the C statement"
        assert elementwise_rel(v[5], v2_[5]) <= 1e-12      # x
        assert elementwise_rel(v[4], v2_[4]) <= 1e-12      # w


def test_bounded_wait_reports_timeout_and_context_survives():
    """A device-side wait that can never be satisfied must end by itself, surface
    as PGB200_ERR_TIMEOUT on the host, and leave the GPU usable."""
    lib = pgb.load()
    assert lib.pgb200SelfTestWaitTimeout(None, 2_000_000) == pgb.OK   # ~1 ms
    torch.cuda.synchronize()
    assert lib.pgb200PollDeviceStatus() == pgb.ERR_TIMEOUT
    assert b"code 99" in lib.pgb200GetLastErrorString()
    assert lib.pgb200PollDeviceStatus() == pgb.OK                      # cleared by the read
    A = dev_fill(128, 64, torch.float64, 1, -1.0, 1.0)
    B = dev_fill(64, 128, torch.float64, 2, -1.0, 1.0)
    Cm = torch.zeros((128, 128), dtype=torch.float64, device=DEV)
    pgb.gemm(1.0, A, B, 0.0, Cm)
    sync_ok()
    assert float((Cm - A @ B).abs().max()) <= 1e-12


@pytest.mark.parametrize("np_dtype", [np.float64, np.float32])
@pytest.mark.parametrize("beta", [1.2, 0.0])
def test_large_host_array_gemm_is_pipelined_and_correct(np_dtype, beta):
    """Host arrays above the pipelining threshold: rows of A and C travel in
    blocks beside the products; the result must equal the oracle's."""
    M, N, K = 2304, 1000, 520          # M not a multiple of the block height, padded pitches
    lo = -1.0 if np_dtype == np.float64 else 0.0
    A = pbo.fill(M, K, np_dtype, SEED, 1, lo, 1.0)
    B = pbo.fill(K, N, np_dtype, SEED, 2, lo, 1.0)
    C0 = pbo.fill(M, N, np_dtype, SEED, 3, lo, 1.0)
    got = C0.copy() if beta else np.full_like(C0, np.nan)
    polybench.kernel_gemm(M, N, K, 1.5, beta, got, A, B)
    pgb.poll_device_status()
    rows = [0, 1, 127, 128, 1151, 1152, M - 1]
    for r in rows:
        ref = pbo.gemm(1.5, beta, C0[r:r + 1].copy(), A[r:r + 1], B)
        if np_dtype == np.float64:
            assert normwise(got[r:r + 1], ref) <= 1e-12
        else:
            assert elementwise_rel(got[r:r + 1], ref) <= 1e-5
    truth = 1.5 * (A.astype(np.float64) @ B.astype(np.float64)) + beta * (C0.astype(np.float64) if beta else 0.0)
    assert normwise(got, truth) <= (1e-12 if np_dtype == np.float64 else 1e-5)


def test_concurrent_host_threads_on_their_own_streams():
    """Generated code may call from OpenMP worker threads: two threads, each on
    its own stream, interleave fp64/fp32 GEMMs and the fused mat-vec (all of
    which use per-stream scratch) and must both get the right answers."""
    import threading
    errs = []

    def worker(tid):
        try:
            torch.cuda.set_device(0)
            st = torch.cuda.Stream()
            with torch.cuda.stream(st):
                n = 384 + 128 * tid
                A = dev_fill(n, n, torch.float64, 10 + tid, -1.0, 1.0)
                B = dev_fill(n, n, torch.float64, 20 + tid, -1.0, 1.0)
                A32 = dev_fill(n, n, torch.float32, 30 + tid, 0.0, 1.0)
                B32 = dev_fill(n, n, torch.float32, 40 + tid, 0.0, 1.0)
                x = dev_fill(1, n, torch.float64, 50 + tid, 0.0, 1.0).reshape(n).contiguous()
                for _ in range(5):
                    Cm = torch.zeros((n, n), dtype=torch.float64, device=DEV)
                    C32 = torch.zeros((n, n), dtype=torch.float32, device=DEV)
                    y1 = torch.zeros(n, dtype=torch.float64, device=DEV)
                    y2 = torch.zeros(n, dtype=torch.float64, device=DEV)
                    pgb.gemm(1.0, A, B, 0.0, Cm, stream=st)
                    pgb.gemm(1.0, A32, B32, 0.0, C32, stream=st)
                    pgb.gemv_pair(1.0, A, x, x, 0.0, y1, y2, stream=st)
                    st.synchronize()
                    assert float((Cm - A @ B).abs().max() / (A @ B).abs().max()) <= 1e-12
                    t32 = A32.double() @ B32.double()
                    assert float(((C32.double() - t32).abs() / t32).max()) <= 1e-5
                    assert float((y1 - A @ x).abs().max() / (A @ x).abs().max()) <= 1e-12
                    assert float((y2 - A.T @ x).abs().max() / (A.T @ x).abs().max()) <= 1e-12
        except Exception as e:  # surfaced in the main thread
            errs.append((tid, repr(e)))

    ts = [threading.Thread(target=worker, args=(t,)) for t in range(2)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert not errs, errs
    pgb.poll_device_status()


@pytest.mark.parametrize("ndev", [1, 2])
def test_single_process_multi_gpu_entries(ndev):
    """pgb200{D,S}gemmMg / pgb200SsyrkMg: row blocks on `ndev` GPUs driven by one
    host thread, shared operand broadcast by NCCL in K-slices."""
    if torch.cuda.device_count() < ndev:
        pytest.skip(f"needs {ndev} GPUs")
    M, N, K = 1100, 520, 2304            # K >= 2048: several K-slices
    A = pbo.fill(M, K, np.float64, SEED, 1, -1.0, 1.0)
    B = pbo.fill(K, N, np.float64, SEED, 2, -1.0, 1.0)
    C0 = pbo.fill(M, N, np.float64, SEED, 3, -1.0, 1.0)
    got = C0.copy()
    pgb.gemm_mg(ndev, 1.5, A, B, 1.2, got)
    assert normwise(got, 1.5 * (A @ B) + 1.2 * C0) <= 1e-12
    for r in (0, 511, 512, M - 1):
        ref = pbo.gemm(1.5, 1.2, C0[r:r + 1].copy(), A[r:r + 1], B)
        assert normwise(got[r:r + 1], ref) <= 1e-12
    A32 = pbo.fill(M, K, np.float32, SEED, 4, 0.0, 1.0)
    B32 = pbo.fill(K, N, np.float32, SEED, 5, 0.0, 1.0)
    C32 = pbo.fill(M, N, np.float32, SEED, 6, 0.0, 1.0)
    got32 = C32.copy()
    pgb.gemm_mg(ndev, 1.5, A32, B32, 1.2, got32)
    t = 1.5 * (A32.astype(np.float64) @ B32.astype(np.float64)) + 1.2 * C32
    assert elementwise_rel(got32, t) <= 1e-5
    n, k = 1300, 2100
    As = pbo.fill(n, k, np.float32, SEED, 7, 0.0, 1.0)
    Cs = pbo.fill(n, n, np.float32, SEED, 8, 0.0, 1.0)
    gots = Cs.copy()
    pgb.syrk_mg(ndev, 1.5, As, 1.2, gots)
    ts = 1.5 * (As.astype(np.float64) @ As.astype(np.float64).T) + 1.2 * Cs
    il, iu = np.tril_indices(n), np.triu_indices(n, 1)
    assert elementwise_rel(gots[il], ts[il]) <= 1e-5
    assert np.array_equal(gots[iu], Cs[iu])
    torch.cuda.set_device(0)
    pgb.poll_device_status()


def test_host_and_device_operands_can_be_mixed():
    M, N, K = 96, 64, 48
    A = dev_fill(M, K, torch.float64, 1, -1.0, 1.0)
    hB = pbo.fill(K, N, np.float64, SEED, 2, -1.0, 1.0)
    hC = pbo.fill(M, N, np.float64, SEED, 3, -1.0, 1.0)
    ref = pbo.gemm(1.5, 1.2, hC.copy(), np.ascontiguousarray(A.cpu().numpy()), hB)
    pgb.gemm(1.5, A, hB, 1.2, hC)  # returns after the copy-back
    assert normwise(hC, ref) <= 1e-12
