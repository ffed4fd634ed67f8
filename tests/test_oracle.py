"""CPU tests of the oracle itself: it must reproduce the reference's golden
dumps and, when the compiled reference kernels are present, match them bit
for bit on seeded inputs."""
import numpy as np
import pytest

from helpers import (MINI, SEED, assert_dump_equal, init_2mm, init_3mm, init_atax, init_bicg,
                     init_doitgen, init_gemm, init_gemver, init_gesummv, init_mvt, init_symm,
                     init_syr2k, init_syrk, init_trmm,
                     read_dump)
from oracle import pbo, ref

TYPES = [("f64", np.float64), ("f32", np.float32)]


@pytest.mark.parametrize("tname,dtype", TYPES)
def test_gemm_golden(tname, dtype):
    ni, nj, nk = MINI["gemm"]
    alpha, beta, C, A, B = init_gemm(ni, nj, nk, dtype)
    pbo.gemm(alpha, beta, C, A, B)
    assert_dump_equal(read_dump("gemm", tname)["C"], C)


@pytest.mark.parametrize("tname,dtype", TYPES)
def test_2mm_golden(tname, dtype):
    ni, nj, nk, nl = MINI["2mm"]
    alpha, beta, tmp, A, B, C, D = init_2mm(ni, nj, nk, nl, dtype)
    pbo.mm2(alpha, beta, tmp, A, B, C, D)
    assert_dump_equal(read_dump("2mm", tname)["D"], D)


@pytest.mark.parametrize("tname,dtype", TYPES)
def test_mvt_golden(tname, dtype):
    (n,) = MINI["mvt"]
    x1, x2, y1, y2, A = init_mvt(n, dtype)
    pbo.mvt(x1, x2, y1, y2, A)
    d = read_dump("mvt", tname)
    assert_dump_equal(d["x1"], x1)
    assert_dump_equal(d["x2"], x2)


@pytest.mark.parametrize("tname,dtype", TYPES)
def test_syrk_golden(tname, dtype):
    n, m = MINI["syrk"]
    alpha, beta, C, A = init_syrk(n, m, dtype)
    C0 = C.copy()
    pbo.syrk(alpha, beta, C, A)
    assert_dump_equal(read_dump("syrk", tname)["C"], C)
    iu = np.triu_indices(n, 1)
    assert np.array_equal(C[iu], C0[iu]), "strict upper triangle must stay untouched"


@pytest.mark.parametrize("tname,dtype", TYPES)
def test_3mm_atax_bicg_gesummv_golden(tname, dtype):
    E, A, B, F, C, D, G = init_3mm(*MINI["3mm"], dtype)
    pbo.mm3(E, A, B, F, C, D, G)
    assert_dump_equal(read_dump("3mm", tname)["G"], G)
    A, x, y, tmp = init_atax(*MINI["atax"], dtype)
    pbo.atax(A, x, y, tmp)
    assert_dump_equal(read_dump("atax", tname)["y"], y)
    A, s, q, p, r = init_bicg(*MINI["bicg"], dtype)
    pbo.bicg(A, s, q, p, r)
    d = read_dump("bicg", tname)
    assert_dump_equal(d["s"], s)
    assert_dump_equal(d["q"], q)
    alpha, beta, A, B, tmp, x, y = init_gesummv(*MINI["gesummv"], dtype)
    pbo.gesummv(alpha, beta, A, B, tmp, x, y)
    assert_dump_equal(read_dump("gesummv", tname)["y"], y)
    alpha, beta, Cm, A, B = init_syr2k(*MINI["syr2k"], dtype)
    pbo.syr2k(alpha, beta, Cm, A, B)
    assert_dump_equal(read_dump("syr2k", tname)["C"], Cm)
    alpha, beta, A, u1, v1, u2, v2, w, x, y, z = init_gemver(*MINI["gemver"], dtype)
    pbo.gemver(alpha, beta, A, u1, v1, u2, v2, w, x, y, z)
    assert_dump_equal(read_dump("gemver", tname)["w"], w)


@pytest.mark.parametrize("tname,dtype", TYPES)
def test_symm_trmm_doitgen_golden(tname, dtype):
    m, n = MINI["symm"]
    alpha, beta, Cm, A, B = init_symm(m, n, dtype)
    pbo.symm(alpha, beta, Cm, A, B)
    assert_dump_equal(read_dump("symm", tname)["C"], Cm)
    m, n = MINI["trmm"]
    alpha, A, B = init_trmm(m, n, dtype)
    pbo.trmm(alpha, A, B)
    assert_dump_equal(read_dump("trmm", tname)["B"], B)
    nr, nq, np_ = MINI["doitgen"]
    A, C4, sum_ = init_doitgen(nr, nq, np_, dtype)
    pbo.doitgen(A, C4, sum_)
    assert_dump_equal(read_dump("doitgen", tname)["A"], A)
    assert np.array_equal(sum_, A[-1, -1]), "sum keeps the last row's result"


needs_ref = pytest.mark.skipif(not ref.available(), reason="compiled reference kernels absent")


def _rand(shape, dtype, aid, lo=-1.0, hi=1.0):
    return pbo.fill(shape[0], shape[1], dtype, SEED, aid, lo, hi)


@needs_ref
@pytest.mark.parametrize("tname,dtype", TYPES)
def test_oracle_matches_compiled_reference(tname, dtype):
    # The reference library is built with FMA contraction allowed, the oracle
    # without; sums of products may differ in the last bits, never more.
    tol = 1e-13 if dtype == np.float64 else 2e-5
    ni, nj, nk, nl = 37, 53, 61, 29
    A, B, C = _rand((ni, nk), dtype, 1), _rand((nk, nj), dtype, 2), _rand((ni, nj), dtype, 3)
    C2 = C.copy()
    pbo.gemm(1.5, 1.2, C, A, B)
    ref.kernel_gemm(ni, nj, nk, 1.5, 1.2, C2, A, B)
    assert np.max(np.abs(C - C2)) <= tol * np.max(np.abs(C2))

    Cc, D = _rand((nj, nl), dtype, 4), _rand((ni, nl), dtype, 5)
    D2 = D.copy()
    tmp, tmp2 = np.zeros((ni, nj), dtype), np.zeros((ni, nj), dtype)
    pbo.mm2(1.5, 1.2, tmp, A, B, Cc, D)
    ref.kernel_2mm(ni, nj, nk, nl, 1.5, 1.2, tmp2, A, B, Cc, D2)
    assert np.max(np.abs(D - D2)) <= tol * np.max(np.abs(D2))
    assert np.max(np.abs(tmp - tmp2)) <= tol * np.max(np.abs(tmp2))

    n = 67
    Am = _rand((n, n), dtype, 6, 0.0, 1.0)
    v = [pbo.fill_vec(n, dtype, SEED, 7 + k, 0.0, 1.0) for k in range(4)]
    w = [x.copy() for x in v]
    pbo.mvt(v[0], v[1], v[2], v[3], Am)
    ref.kernel_mvt(n, w[0], w[1], w[2], w[3], Am)
    for a, b in zip(v[:2], w[:2]):
        assert np.max(np.abs(a - b)) <= tol * np.max(np.abs(b))

    n, m = 45, 33
    As, Cs = _rand((n, m), dtype, 11), _rand((n, n), dtype, 12)
    Cs2 = Cs.copy()
    pbo.syrk(1.5, 1.2, Cs, As)
    ref.kernel_syrk(n, m, 1.5, 1.2, Cs2, As)
    assert np.max(np.abs(Cs - Cs2)) <= tol * np.max(np.abs(Cs2))


@needs_ref
@pytest.mark.parametrize("tname,dtype", TYPES)
def test_oracle_matches_compiled_reference_symm_trmm_doitgen(tname, dtype):
    tol = 1e-13 if dtype == np.float64 else 2e-5
    m, n = 43, 37
    A, B, Cm = _rand((m, m), dtype, 21), _rand((m, n), dtype, 22), _rand((m, n), dtype, 23)
    A[np.triu_indices(m, 1)] = -999  # must never be read
    C2 = Cm.copy()
    pbo.symm(1.5, 1.2, Cm, A, B)
    ref.kernel_symm(m, n, 1.5, 1.2, C2, A, B)
    assert np.max(np.abs(Cm - C2)) <= tol * np.max(np.abs(C2))

    B1, B2 = B.copy(), B.copy()
    pbo.trmm(1.5, A, B1)
    ref.kernel_trmm(m, n, 1.5, A, B2)
    assert np.max(np.abs(B1 - B2)) <= tol * np.max(np.abs(B2))
    assert np.max(np.abs(B2)) < 1e3, "the sentinel in A's upper triangle leaked into the result"

    nr, nq, np_ = 5, 7, 19
    A3 = _rand((nr * nq, np_), dtype, 24).reshape(nr, nq, np_)
    C4 = _rand((np_, np_), dtype, 25)
    A4 = A3.copy()
    s1, s2 = np.zeros(np_, dtype), np.zeros(np_, dtype)
    pbo.doitgen(A3, C4, s1)
    ref.kernel_doitgen(nr, nq, np_, A4, C4, s2)
    assert np.max(np.abs(A3 - A4)) <= tol * np.max(np.abs(A4))


@needs_ref
@pytest.mark.parametrize("tname,dtype", TYPES)
def test_oracle_matches_compiled_reference_widened_nests(tname, dtype):
    """3mm, atax, bicg, gesummv, syr2k and gemver on seeded random inputs against
    the reference's own compiled kernels (FMA contraction may differ, no more)."""
    tol = 1e-13 if dtype == np.float64 else 2e-5

    def close(a, b):
        return np.max(np.abs(a - b)) <= tol * max(np.max(np.abs(b)), 1e-30)

    ni, nj, nk, nl, nm = 13, 17, 19, 23, 11
    A, B = _rand((ni, nk), dtype, 31), _rand((nk, nj), dtype, 32)
    Cm, D = _rand((nj, nm), dtype, 33), _rand((nm, nl), dtype, 34)
    out1 = [np.zeros(s_, dtype) for s_ in ((ni, nj), (nj, nl), (ni, nl))]
    out2 = [o.copy() for o in out1]
    pbo.mm3(out1[0], A, B, out1[1], Cm, D, out1[2])
    ref.kernel_3mm(ni, nj, nk, nl, nm, out2[0], A, B, out2[1], Cm, D, out2[2])
    assert all(close(a, b) for a, b in zip(out1, out2))

    m, n = 21, 27
    Am, x = _rand((m, n), dtype, 35), pbo.fill_vec(n, dtype, SEED, 36, 0.0, 1.0)
    y1, t1, y2, t2 = (np.zeros(k, dtype) for k in (n, m, n, m))
    pbo.atax(Am, x, y1, t1)
    ref.kernel_atax(m, n, Am, x, y2, t2)
    assert close(y1, y2) and close(t1, t2)

    Ab = _rand((n, m), dtype, 37)                       # bicg: A is n x m
    p_, r_ = pbo.fill_vec(m, dtype, SEED, 38, 0.0, 1.0), pbo.fill_vec(n, dtype, SEED, 39, 0.0, 1.0)
    s1, q1, s2, q2 = (np.zeros(k, dtype) for k in (m, n, m, n))
    pbo.bicg(Ab, s1, q1, p_, r_)
    ref.kernel_bicg(m, n, Ab, s2, q2, p_, r_)
    assert close(s1, s2) and close(q1, q2)

    n = 31
    Ag, Bg = _rand((n, n), dtype, 40), _rand((n, n), dtype, 41)
    xg = pbo.fill_vec(n, dtype, SEED, 42, 0.0, 1.0)
    ya, ta, yb, tb = (np.zeros(n, dtype) for _ in range(4))
    pbo.gesummv(1.5, 1.2, Ag, Bg, ta, xg, ya)
    ref.kernel_gesummv(n, 1.5, 1.2, Ag, Bg, tb, xg, yb)
    assert close(ya, yb) and close(ta, tb)

    n, m = 26, 18
    As, Bs, Cs = _rand((n, m), dtype, 43), _rand((n, m), dtype, 44), _rand((n, n), dtype, 45)
    Cs2 = Cs.copy()
    pbo.syr2k(1.5, 1.2, Cs, As, Bs)
    ref.kernel_syr2k(n, m, 1.5, 1.2, Cs2, As, Bs)
    assert close(Cs, Cs2)

    n = 33
    Av = _rand((n, n), dtype, 46)
    vec = [pbo.fill_vec(n, dtype, SEED, 47 + k, 0.0, 1.0) for k in range(8)]
    Av2, vec2 = Av.copy(), [v.copy() for v in vec]
    pbo.gemver(1.5, 1.2, Av, *vec)
    ref.kernel_gemver(n, 1.5, 1.2, Av2, *vec2)
    assert close(Av, Av2) and all(close(a, b) for a, b in zip(vec, vec2))


def test_symm_trmm_doitgen_closed_forms():
    """What the three nests compute, stated as matrix algebra (the device code
    implements these forms, the oracle the loop nests): they must agree."""
    rng = np.random.default_rng(11)
    m, n = 37, 29
    A = rng.uniform(0, 1, (m, m))
    B = rng.uniform(0, 1, (m, n))
    Cm = rng.uniform(0, 1, (m, n))
    L = np.tril(A)
    S = L + np.tril(A, -1).T                       # symmetric, from the lower triangle
    got = pbo.symm(1.5, 1.2, Cm.copy(), np.where(np.tri(m, dtype=bool), A, np.nan), B)
    assert np.allclose(got, 1.2 * Cm + 1.5 * S @ B, rtol=1e-13, atol=0)
    U = np.eye(m) + np.tril(A, -1).T               # unit upper triangular
    got = pbo.trmm(1.5, np.where(np.tri(m, k=-1, dtype=bool), A, np.nan), B.copy())
    assert np.allclose(got, 1.5 * U @ B, rtol=1e-13, atol=0)
    nr, nq, np_ = 4, 5, 13
    A3 = rng.uniform(-1, 1, (nr, nq, np_))
    C4 = rng.uniform(-1, 1, (np_, np_))
    s_ = np.zeros(np_)
    got = pbo.doitgen(A3.copy(), C4, s_)
    assert np.allclose(got, A3 @ C4, rtol=1e-12, atol=1e-14)
    assert np.array_equal(s_, got[-1, -1])


def test_row_restricted_oracle_is_bit_identical():
    n, m = 40, 24
    A, C = _rand((n, m), np.float64, 1), _rand((n, n), np.float64, 2)
    full = pbo.syrk(1.5, 1.2, C.copy(), A)
    part = C.copy()
    pbo.syrk(1.5, 1.2, part, A, 10, 25)
    assert np.array_equal(part[10:25], full[10:25])
    assert np.array_equal(part[:10], C[:10]) and np.array_equal(part[25:], C[25:])

    Am = _rand((n, n), np.float64, 3, 0.0, 1.0)
    v = [pbo.fill_vec(n, np.float64, SEED, 4 + k, 0.0, 1.0) for k in range(4)]
    f = [x.copy() for x in v]
    pbo.mvt(f[0], f[1], f[2], f[3], Am)
    p = [x.copy() for x in v]
    pbo.mvt(p[0], p[1], p[2], p[3], Am, 5, 17)
    assert np.array_equal(p[0][5:17], f[0][5:17]) and np.array_equal(p[1][5:17], f[1][5:17])


def test_generator_properties():
    a = pbo.fill(64, 48, np.float64, SEED, 1, -1.0, 1.0)
    assert a.min() >= -1.0 and a.max() < 1.0 and abs(a.mean()) < 0.05
    # counter-based: a row block generated on its own equals the same rows of the whole
    b = pbo.fill(16, 48, np.float64, SEED, 1, -1.0, 1.0, row0=20)
    assert np.array_equal(b, a[20:36])
    # padded destination leaves the padding alone
    buf = np.full((8, 20), 7.0, dtype=np.float32)
    pbo.fill(8, 16, np.float32, SEED, 2, 0.0, 1.0, out=buf[:, :16])
    assert np.all(buf[:, 16:] == 7.0) and buf[:, :16].max() < 1.0 and buf[:, :16].min() >= 0.0
    c = pbo.fill(8, 16, np.float32, SEED, 3, 0.0, 1.0)
    assert not np.array_equal(c, buf[:, :16])
    # acc64 variant agrees with a numpy float64 evaluation
    A = pbo.fill(9, 13, np.float32, SEED, 4, 0.0, 1.0)
    B = pbo.fill(13, 11, np.float32, SEED, 5, 0.0, 1.0)
    Cm = pbo.fill(9, 11, np.float32, SEED, 6, 0.0, 1.0)
    t = pbo.gemm_acc64(1.5, 1.2, Cm, A, B)
    e = np.float64(np.float32(1.5)) * (A.astype(np.float64) @ B.astype(np.float64)) + \
        np.float64(np.float32(1.2)) * Cm.astype(np.float64)
    assert np.max(np.abs(t - e)) < 1e-12
