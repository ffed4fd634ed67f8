"""Shared test helpers: PolyBench's deterministic init formulas, the dump text
format of the reference's verification executables, and error metrics."""
import os
import re

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
SEED = 20261125


# ---------------------------------------------------------------------------
# init_array of each kernel (the reference's formulas, restated):
#   gemm.c:42-63, 2mm.c:41-67, mvt.c:39-58, syrk.c:39-56
# `(DATA_TYPE)(int expr) / n`: integer expression, converted, divided in
# DATA_TYPE arithmetic.
# ---------------------------------------------------------------------------
def _grid(r, c):
    return np.arange(r, dtype=np.int64)[:, None], np.arange(c, dtype=np.int64)[None, :]


def init_gemm(ni, nj, nk, dtype):
    dt = np.dtype(dtype).type
    i, j = _grid(ni, nj)
    C = ((i * j + 1) % ni).astype(dtype) / dt(ni)
    i, j = _grid(ni, nk)
    A = (i * (j + 1) % nk).astype(dtype) / dt(nk)
    i, j = _grid(nk, nj)
    B = (i * (j + 2) % nj).astype(dtype) / dt(nj)
    return dt(1.5), dt(1.2), C, A, B


def init_2mm(ni, nj, nk, nl, dtype):
    dt = np.dtype(dtype).type
    i, j = _grid(ni, nk)
    A = ((i * j + 1) % ni).astype(dtype) / dt(ni)
    i, j = _grid(nk, nj)
    B = (i * (j + 1) % nj).astype(dtype) / dt(nj)
    i, j = _grid(nj, nl)
    C = ((i * (j + 3) + 1) % nl).astype(dtype) / dt(nl)
    i, j = _grid(ni, nl)
    D = (i * (j + 2) % nk).astype(dtype) / dt(nk)
    tmp = np.zeros((ni, nj), dtype=dtype)
    return dt(1.5), dt(1.2), tmp, A, B, C, D


def init_mvt(n, dtype):
    dt = np.dtype(dtype).type
    i = np.arange(n, dtype=np.int64)
    x1 = (i % n).astype(dtype) / dt(n)
    x2 = ((i + 1) % n).astype(dtype) / dt(n)
    y1 = ((i + 3) % n).astype(dtype) / dt(n)
    y2 = ((i + 4) % n).astype(dtype) / dt(n)
    ii, jj = _grid(n, n)
    A = (ii * jj % n).astype(dtype) / dt(n)
    return x1, x2, y1, y2, A


def init_syrk(n, m, dtype):
    dt = np.dtype(dtype).type
    i, j = _grid(n, m)
    A = ((i * j + 1) % n).astype(dtype) / dt(n)
    i, j = _grid(n, n)
    C = ((i * j + 2) % m).astype(dtype) / dt(m)
    return dt(1.5), dt(1.2), C, A


def init_3mm(ni, nj, nk, nl, nm, dtype):
    """3mm.c:41-62"""
    dt = np.dtype(dtype).type
    i, j = _grid(ni, nk)
    A = ((i * j + 1) % ni).astype(dtype) / dt(5 * ni)
    i, j = _grid(nk, nj)
    B = ((i * (j + 1) + 2) % nj).astype(dtype) / dt(5 * nj)
    i, j = _grid(nj, nm)
    C = (i * (j + 3) % nl).astype(dtype) / dt(5 * nl)
    i, j = _grid(nm, nl)
    D = ((i * (j + 2) + 2) % nk).astype(dtype) / dt(5 * nk)
    E, F, G = (np.zeros(s, dtype=dtype) for s in ((ni, nj), (nj, nl), (ni, nl)))
    return E, A, B, F, C, D, G


def init_atax(m, n, dtype):
    """atax.c:40-54"""
    dt = np.dtype(dtype).type
    x = dt(1) + np.arange(n).astype(dtype) / dt(n)
    i, j = _grid(m, n)
    A = ((i + j) % n).astype(dtype) / dt(5 * m)
    return A, x.astype(dtype), np.zeros(n, dtype=dtype), np.zeros(m, dtype=dtype)


def init_bicg(m, n, dtype):
    """bicg.c:40-54 (A is n x m)"""
    dt = np.dtype(dtype).type
    p = (np.arange(m) % m).astype(dtype) / dt(m)
    r = (np.arange(n) % n).astype(dtype) / dt(n)
    i, j = _grid(n, m)
    A = (i * (j + 1) % n).astype(dtype) / dt(n)
    return A, np.zeros(m, dtype=dtype), np.zeros(n, dtype=dtype), p, r


def init_gesummv(n, dtype):
    """gesummv.c:40-58"""
    dt = np.dtype(dtype).type
    x = (np.arange(n) % n).astype(dtype) / dt(n)
    i, j = _grid(n, n)
    A = ((i * j + 1) % n).astype(dtype) / dt(n)
    B = ((i * j + 2) % n).astype(dtype) / dt(n)
    return dt(1.5), dt(1.2), A, B, np.zeros(n, dtype=dtype), x, np.zeros(n, dtype=dtype)


def init_syr2k(n, m, dtype):
    """syr2k.c:40-60"""
    dt = np.dtype(dtype).type
    i, j = _grid(n, m)
    A = ((i * j + 1) % n).astype(dtype) / dt(n)
    B = ((i * j + 2) % m).astype(dtype) / dt(m)
    i, j = _grid(n, n)
    C = ((i * j + 3) % n).astype(dtype) / dt(m)
    return dt(1.5), dt(1.2), C, A, B


def init_gemver(n, dtype):
    """gemver.c:40-73"""
    dt = np.dtype(dtype).type
    i = np.arange(n)
    f = (i + 1).astype(dtype) / dt(n)
    u1 = i.astype(dtype)
    u2, v1, v2, y, z = f / dt(2.0), f / dt(4.0), f / dt(6.0), f / dt(8.0), f / dt(9.0)
    ii, jj = _grid(n, n)
    A = (ii * jj % n).astype(dtype) / dt(n)
    return (dt(1.5), dt(1.2), A, u1, v1.astype(dtype), u2.astype(dtype), v2.astype(dtype),
            np.zeros(n, dtype=dtype), np.zeros(n, dtype=dtype), y.astype(dtype), z.astype(dtype))


def init_symm(m, n, dtype):
    """symm.c:41-63 (the strict upper triangle of A holds the -999 sentinel)"""
    dt = np.dtype(dtype).type
    i, j = _grid(m, n)
    C = ((i + j) % 100).astype(dtype) / dt(m)
    B = ((n + i - j) % 100).astype(dtype) / dt(m)
    i, j = _grid(m, m)
    A = np.where(j <= i, ((i + j) % 100).astype(dtype) / dt(m), dt(-999)).astype(dtype)
    return dt(1.5), dt(1.2), C, A, B


def init_trmm(m, n, dtype):
    """trmm.c:41-59 (the strict upper triangle of A is left untouched by the
    reference; zero here, never read by the nest)"""
    dt = np.dtype(dtype).type
    i, j = _grid(m, m)
    A = np.where(j < i, ((i + j) % m).astype(dtype) / dt(m), dt(0)).astype(dtype)
    A[np.arange(m), np.arange(m)] = dt(1)
    i, j = _grid(m, n)
    B = ((n + (i - j)) % n).astype(dtype) / dt(n)
    return dt(1.5), A, B


def init_doitgen(nr, nq, np_, dtype):
    """doitgen.c:41-54"""
    dt = np.dtype(dtype).type
    i, j, k = np.meshgrid(np.arange(nr), np.arange(nq), np.arange(np_), indexing="ij")
    A = ((i * j + k) % np_).astype(dtype) / dt(np_)
    i, j = _grid(np_, np_)
    C4 = (i * j % np_).astype(dtype) / dt(np_)
    return np.ascontiguousarray(A), C4, np.zeros(np_, dtype=dtype)


MINI = {"symm": (20, 30), "trmm": (20, 30), "doitgen": (10, 8, 12),  # doitgen: (NR, NQ, NP)
        "gemver": (40,), "syr2k": (30, 20), "3mm": (16, 18, 20, 22, 24), "atax": (38, 42), "bicg": (38, 42), "gesummv": (30,),
        "gemm": (20, 25, 30), "2mm": (16, 18, 22, 24), "mvt": (40,), "syrk": (30, 20)}  # syrk: (N, M)


def read_dump(kernel, tname):
    """Parse tests/golden/<kernel>_mini_<tname>.dump.txt into {array: [tokens]}."""
    text = open(os.path.join(GOLDEN, f"{kernel}_mini_{tname}.dump.txt")).read()
    out = {}
    for m in re.finditer(r"begin dump: (\w+)(.*?)end\s+dump: \1", text, re.S):
        out[m.group(1)] = m.group(2).split()
    return out


def fmt_tokens(a):
    """DATA_PRINTF_MODIFIER "%0.2lf " applied to every element, row-major."""
    return ["%0.2f" % float(v) for v in np.asarray(a, dtype=np.float64).ravel()]


def assert_dump_equal(tokens, arr, slack_ulps=0):
    got = fmt_tokens(arr)
    assert len(got) == len(tokens)
    bad = [(k, g, t) for k, (g, t) in enumerate(zip(got, tokens)) if g != t]
    if slack_ulps and bad:
        # A different (but valid) summation order may move a value across a
        # 2-decimal rounding boundary; accept only if the values themselves
        # agree to `slack_ulps` in the last printed digit.
        bad = [(k, g, t) for k, g, t in bad if abs(float(g) - float(t)) > 0.011 * slack_ulps]
    assert not bad, f"{len(bad)} dump tokens differ, first: {bad[:5]}"


# ---------------------------------------------------------------------------
# error metrics
# ---------------------------------------------------------------------------
def normwise(got, ref):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.max(np.abs(got - ref)) / max(np.max(np.abs(ref)), 1e-300))


def elementwise_rel(got, ref):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.maximum(np.abs(ref), 1e-300)
    return float(np.max(np.abs(got - ref) / den))


def backward_gemm(got, ref, alpha, beta, A, B, C0):
    """max |d| / (|alpha||A||B| + |beta||C0|): componentwise backward error."""
    den = abs(alpha) * (np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64))
    den = den + abs(beta) * np.abs(C0).astype(np.float64)
    d = np.abs(np.asarray(got, np.float64) - np.asarray(ref, np.float64))
    return float(np.max(d / np.maximum(den, 1e-300)))
