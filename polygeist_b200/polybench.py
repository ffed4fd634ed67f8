"""Host-array mirror of the reference's PolyBench kernel functions.

Same names, argument order and in-place semantics as
  kernel_gemm  tools/cgeist/Test/polybench/linear-algebra/blas/gemm/gemm.c:88-115
  kernel_2mm   tools/cgeist/Test/polybench/linear-algebra/kernels/2mm/2mm.c:92-121
  kernel_mvt   tools/cgeist/Test/polybench/linear-algebra/kernels/mvt/mvt.c:93-111
  kernel_syrk  tools/cgeist/Test/polybench/linear-algebra/blas/syrk/syrk.c:83-108
and of the same-shaped nests kernel_3mm (kernels/3mm/3mm.c:87-127), kernel_atax
(kernels/atax/atax.c:80-102), kernel_syr2k (blas/syr2k/syr2k.c:84-112), kernel_gemver (blas/gemver/gemver.c:97-133), kernel_bicg (kernels/bicg/bicg.c:86-111) and
kernel_gesummv (blas/gesummv/gesummv.c:86-112).
Arrays are C-contiguous numpy arrays in host memory with exactly the extents
given by the size arguments (the C99-prototype form of the PolyBench
signatures); float64 takes the DATA_TYPE=double build, float32 the
-DDATA_TYPE_IS_FLOAT build.  Each call goes through the library's
`pgb200_kernel_*` drop-in, which stages the operands to the GPU, runs the
contraction and copies the live-out arrays back.
"""
import numpy as np

from . import check, load


def _req(a, shape):
    if not (isinstance(a, np.ndarray) and a.flags["C_CONTIGUOUS"] and tuple(a.shape) == tuple(shape)):
        raise ValueError(f"expected a C-contiguous numpy array of shape {tuple(shape)}")
    return a.ctypes.data


def kernel_gemm(ni, nj, nk, alpha, beta, C, A, B):
    f = load().pgb200_kernel_gemm if C.dtype == np.float64 else load().pgb200_kernel_gemm_f32
    check(f(ni, nj, nk, alpha, beta, _req(C, (ni, nj)), _req(A, (ni, nk)), _req(B, (nk, nj))))


def kernel_2mm(ni, nj, nk, nl, alpha, beta, tmp, A, B, C, D):
    if D.dtype != np.float64:
        raise ValueError("kernel_2mm: float64 only")
    check(load().pgb200_kernel_2mm(ni, nj, nk, nl, alpha, beta, _req(tmp, (ni, nj)),
                                   _req(A, (ni, nk)), _req(B, (nk, nj)), _req(C, (nj, nl)),
                                   _req(D, (ni, nl))))


def kernel_mvt(n, x1, x2, y_1, y_2, A):
    if A.dtype != np.float64:
        raise ValueError("kernel_mvt: float64 only")
    check(load().pgb200_kernel_mvt(n, _req(x1, (n,)), _req(x2, (n,)), _req(y_1, (n,)),
                                   _req(y_2, (n,)), _req(A, (n, n))))


def kernel_syrk(n, m, alpha, beta, C, A):
    f = load().pgb200_kernel_syrk if C.dtype == np.float64 else load().pgb200_kernel_syrk_f32
    check(f(n, m, alpha, beta, _req(C, (n, n)), _req(A, (n, m))))


def _f64(*arrs):
    for a in arrs:
        if a.dtype != np.float64:
            raise ValueError("float64 only")


def kernel_3mm(ni, nj, nk, nl, nm, E, A, B, F, C, D, G):
    _f64(E, A, B, F, C, D, G)
    check(load().pgb200_kernel_3mm(ni, nj, nk, nl, nm, _req(E, (ni, nj)), _req(A, (ni, nk)),
                                   _req(B, (nk, nj)), _req(F, (nj, nl)), _req(C, (nj, nm)),
                                   _req(D, (nm, nl)), _req(G, (ni, nl))))


def kernel_atax(m, n, A, x, y, tmp):
    _f64(A, x, y, tmp)
    check(load().pgb200_kernel_atax(m, n, _req(A, (m, n)), _req(x, (n,)), _req(y, (n,)),
                                    _req(tmp, (m,))))


def kernel_bicg(m, n, A, s, q, p, r):
    _f64(A, s, q, p, r)
    check(load().pgb200_kernel_bicg(m, n, _req(A, (n, m)), _req(s, (m,)), _req(q, (n,)),
                                    _req(p, (m,)), _req(r, (n,))))


def kernel_gesummv(n, alpha, beta, A, B, tmp, x, y):
    _f64(A, B, tmp, x, y)
    check(load().pgb200_kernel_gesummv(n, alpha, beta, _req(A, (n, n)), _req(B, (n, n)),
                                       _req(tmp, (n,)), _req(x, (n,)), _req(y, (n,))))


def kernel_syr2k(n, m, alpha, beta, C, A, B):
    f = load().pgb200_kernel_syr2k if C.dtype == np.float64 else load().pgb200_kernel_syr2k_f32
    check(f(n, m, alpha, beta, _req(C, (n, n)), _req(A, (n, m)), _req(B, (n, m))))


def kernel_gemver(n, alpha, beta, A, u1, v1, u2, v2, w, x, y, z):
    _f64(A, u1, v1, u2, v2, w, x, y, z)
    vecs = [_req(v, (n,)) for v in (u1, v1, u2, v2, w, x, y, z)]
    check(load().pgb200_kernel_gemver(n, alpha, beta, _req(A, (n, n)), *vecs))


def kernel_symm(m, n, alpha, beta, C, A, B):
    f = load().pgb200_kernel_symm if C.dtype == np.float64 else load().pgb200_kernel_symm_f32
    check(f(m, n, alpha, beta, _req(C, (m, n)), _req(A, (m, m)), _req(B, (m, n))))


def kernel_trmm(m, n, alpha, A, B):
    f = load().pgb200_kernel_trmm if B.dtype == np.float64 else load().pgb200_kernel_trmm_f32
    check(f(m, n, alpha, _req(A, (m, m)), _req(B, (m, n))))


def kernel_doitgen(nr, nq, np_, A, C4, sum_):
    _f64(A, C4, sum_)
    check(load().pgb200_kernel_doitgen(nr, nq, np_, _req(A, (nr, nq, np_)), _req(C4, (np_, np_)),
                                       _req(sum_, (np_,))))
