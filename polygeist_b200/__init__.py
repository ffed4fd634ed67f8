"""polygeist_b200 - Python host side of libpgb200.

The product is the C-ABI shared library (include/pgb200.h).  This package
  * builds / loads it (`load()`), with typed ctypes signatures for every symbol
    the header declares;
  * offers thin array-level wrappers (`dgemm`, `sgemm`, `dsyrk`, `ssyrk`,
    `dgemv`, `dmvt`, `fill_uniform`) that accept torch CUDA tensors (used in
    place) or numpy arrays (host memory, staged by the library);
  * mirrors the reference's PolyBench kernel functions for host arrays in
    `polygeist_b200.polybench` (kernel_gemm, kernel_2mm, kernel_mvt,
    kernel_syrk: same names, argument order and in-place semantics).

There is no CPU fallback: if the library cannot be loaded, or no sm_100 GPU
is present, calls raise.
"""
import ctypes as C
import os

import numpy as np

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libpgb200.so")

OK, ERR_INVALID, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT, ERR_UNSUPPORTED = range(6)
PATH_NONE, PATH_SIMT, PATH_DMMA, PATH_TCGEN05, PATH_STREAM = range(5)


class PGB200Error(RuntimeError):
    def __init__(self, status, msg):
        super().__init__(f"libpgb200 status {status}: {msg}")
        self.status = status


class Config(C.Structure):
    _fields_ = [("log_level", C.c_int32), ("sgemm_chunk_kblocks", C.c_int32),
                ("force_generic", C.c_int32), ("sgemm_planes_only", C.c_int32),
                ("reserve_sms", C.c_int32), ("no_two_cta", C.c_int32),
                ("no_split_k", C.c_int32), ("sgemm_b_in_place", C.c_int32),
                ("no_step_sync", C.c_int32)]


_i32, _i64, _vp, _f64, _f32 = C.c_int32, C.c_int64, C.c_void_p, C.c_double, C.c_float
_int = C.c_int

# name -> (restype, argtypes); must list every symbol of include/pgb200.h.
SIGNATURES = {
    "pgb200Init": (_i32, [C.POINTER(Config)]),
    "pgb200Shutdown": (_i32, []),
    "pgb200GetLastErrorString": (C.c_char_p, []),
    "pgb200Version": (_i32, []),
    "pgb200Dgemm": (_i32, [_vp, _i64, _i64, _i64, _f64, _vp, _i64, _vp, _i64, _f64, _vp, _i64]),
    "pgb200Sgemm": (_i32, [_vp, _i64, _i64, _i64, _f32, _vp, _i64, _vp, _i64, _f32, _vp, _i64]),
    "pgb200DgemmNT": (_i32, [_vp, _i64, _i64, _i64, _f64, _vp, _i64, _vp, _i64, _f64, _vp, _i64]),
    "pgb200SgemmNT": (_i32, [_vp, _i64, _i64, _i64, _f32, _vp, _i64, _vp, _i64, _f32, _vp, _i64]),
    "pgb200Dsyr2k": (_i32, [_vp, _i64, _i64, _f64, _vp, _i64, _vp, _i64, _f64, _vp, _i64]),
    "pgb200Ssyr2k": (_i32, [_vp, _i64, _i64, _f32, _vp, _i64, _vp, _i64, _f32, _vp, _i64]),
    "pgb200DgemmMg": (_i32, [_i32, _i64, _i64, _i64, _f64, _vp, _i64, _vp, _i64, _f64, _vp, _i64]),
    "pgb200SgemmMg": (_i32, [_i32, _i64, _i64, _i64, _f32, _vp, _i64, _vp, _i64, _f32, _vp, _i64]),
    "pgb200SsyrkMg": (_i32, [_i32, _i64, _i64, _f32, _vp, _i64, _f32, _vp, _i64]),
    "pgb200Dsyrk": (_i32, [_vp, _i64, _i64, _f64, _vp, _i64, _f64, _vp, _i64]),
    "pgb200Ssyrk": (_i32, [_vp, _i64, _i64, _f32, _vp, _i64, _f32, _vp, _i64]),
    "pgb200SsyrkRows": (_i32, [_vp, _i64, _i64, _i64, _i64, _f32, _vp, _i64, _f32, _vp, _i64]),
    "pgb200Dgemv": (_i32, [_vp, _i32, _i64, _i64, _f64, _vp, _i64, _vp, _f64, _vp]),
    "pgb200DgemvPair": (_i32, [_vp, _i64, _i64, _f64, _vp, _i64, _vp, _vp, _f64, _vp, _vp]),
    "pgb200Dgemver": (_i32, [_vp, _i64, _f64, _f64, _vp, _i64] + [_vp] * 8),
    "pgb200Dmvt": (_i32, [_vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp]),
    "pgb200DmvtNoAlloc": (_i32, [_vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp]),
    "pgb200FillUniformF64": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, C.c_uint64, C.c_uint32, _f64, _f64]),
    "pgb200FillUniformF32": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, C.c_uint64, C.c_uint32, _f32, _f32]),
    "pgb200Pin": (_i32, [_vp, C.c_uint64]),
    "pgb200PinSync": (_i32, [_vp]),
    "pgb200Unpin": (_i32, [_vp]),
    "pgb200TransferCounters": (_i32, [C.POINTER(_i64), C.POINTER(_i64)]),
    "pgb200ProfileEnable": (_i32, [_i32]),
    "pgb200ProfileDump": (_i32, [C.c_char_p]),
    "pgb200LastPath": (_i32, []),
    "pgb200PollDeviceStatus": (_i32, []),
    "pgb200SelfTestWaitTimeout": (_i32, [_vp, _i64]),
    "pgb200LaunchCount": (_i64, []),
    "pgb200ProbePeak": (_i32, [_vp, _i32, C.POINTER(_f64)]),
    "pgb200_kernel_gemm": (_i32, [_int, _int, _int, _f64, _f64, _vp, _vp, _vp]),
    "pgb200_kernel_gemm_f32": (_i32, [_int, _int, _int, _f32, _f32, _vp, _vp, _vp]),
    "pgb200_kernel_2mm": (_i32, [_int, _int, _int, _int, _f64, _f64, _vp, _vp, _vp, _vp, _vp]),
    "pgb200_kernel_mvt": (_i32, [_int, _vp, _vp, _vp, _vp, _vp]),
    "pgb200_kernel_syrk": (_i32, [_int, _int, _f64, _f64, _vp, _vp]),
    "pgb200_kernel_syrk_f32": (_i32, [_int, _int, _f32, _f32, _vp, _vp]),
    "pgb200_kernel_syr2k": (_i32, [_int, _int, _f64, _f64, _vp, _vp, _vp]),
    "pgb200_kernel_syr2k_f32": (_i32, [_int, _int, _f32, _f32, _vp, _vp, _vp]),
    "pgb200_kernel_gemver": (_i32, [_int, _f64, _f64] + [_vp] * 9),
    "pgb200_kernel_3mm": (_i32, [_int] * 5 + [_vp] * 7),
    "pgb200_kernel_atax": (_i32, [_int, _int, _vp, _vp, _vp, _vp]),
    "pgb200_kernel_bicg": (_i32, [_int, _int, _vp, _vp, _vp, _vp, _vp]),
    "pgb200_kernel_gesummv": (_i32, [_int, _f64, _f64, _vp, _vp, _vp, _vp, _vp]),
    "pgb200Dsymm": (_i32, [_vp, _i64, _i64, _f64, _vp, _i64, _vp, _i64, _f64, _vp, _i64]),
    "pgb200Ssymm": (_i32, [_vp, _i64, _i64, _f32, _vp, _i64, _vp, _i64, _f32, _vp, _i64]),
    "pgb200Dtrmm": (_i32, [_vp, _i64, _i64, _f64, _vp, _i64, _vp, _i64]),
    "pgb200Strmm": (_i32, [_vp, _i64, _i64, _f32, _vp, _i64, _vp, _i64]),
    "pgb200Ddoitgen": (_i32, [_vp, _i64, _i64, _vp, _i64, _vp, _i64, _vp]),
    "pgb200_kernel_symm": (_i32, [_int, _int, _f64, _f64, _vp, _vp, _vp]),
    "pgb200_kernel_symm_f32": (_i32, [_int, _int, _f32, _f32, _vp, _vp, _vp]),
    "pgb200_kernel_trmm": (_i32, [_int, _int, _f64, _vp, _vp]),
    "pgb200_kernel_trmm_f32": (_i32, [_int, _int, _f32, _vp, _vp]),
    "pgb200_kernel_doitgen": (_i32, [_int, _int, _int, _vp, _vp, _vp]),
}

_lib = None


def load(build_if_missing=True):
    """Return the ctypes handle of libpgb200.so (building it in-tree first when
    it is absent and nvcc is available)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        if not build_if_missing:
            raise ImportError(f"{LIB_PATH} is missing; run python -m polygeist_b200.build")
        from . import build as _b
        _b.build()
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header/library mismatch
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status):
    if status != OK:
        raise PGB200Error(status, load().pgb200GetLastErrorString().decode())


def init(log_level=0, sgemm_chunk_kblocks=0, force_generic=0, sgemm_planes_only=0, reserve_sms=0,
         no_two_cta=0, no_split_k=0, sgemm_b_in_place=0, no_step_sync=0):
    cfg = Config(log_level, sgemm_chunk_kblocks, force_generic, sgemm_planes_only, reserve_sms,
                 no_two_cta, no_split_k, sgemm_b_in_place, no_step_sync)
    check(load().pgb200Init(C.byref(cfg)))


def pin(a):
    """Register the host array `a` (numpy): a device copy is made now and used by
    every call that is handed `a` (or a view into it) until unpin(a)."""
    check(load().pgb200Pin(C.c_void_p(a.ctypes.data), C.c_uint64(a.nbytes)))


def pin_sync(a):
    check(load().pgb200PinSync(C.c_void_p(a.ctypes.data)))


def unpin(a):
    check(load().pgb200Unpin(C.c_void_p(a.ctypes.data)))


def transfer_counters():
    """(host->device bytes, device->host bytes) copied by the library so far."""
    h, d = _i64(0), _i64(0)
    check(load().pgb200TransferCounters(C.byref(h), C.byref(d)))
    return h.value, d.value


def profile_enable(on=True):
    check(load().pgb200ProfileEnable(1 if on else 0))


def profile_dump(path=None):
    check(load().pgb200ProfileDump(None if path is None else os.fsencode(path)))


def last_path():
    return load().pgb200LastPath()


def launch_count():
    return load().pgb200LaunchCount()


def poll_device_status():
    check(load().pgb200PollDeviceStatus())


# ---------------------------------------------------------------------------
# array plumbing: torch CUDA tensors or numpy arrays
# ---------------------------------------------------------------------------
def _is_torch(a):
    return type(a).__module__.startswith("torch")


def _ptr(a):
    if a is None:
        return None
    return a.data_ptr() if _is_torch(a) else a.ctypes.data


def _ld(a):
    """Leading dimension (in elements) of a row-major 2-D array/tensor."""
    if _is_torch(a):
        assert a.dim() == 2 and (a.stride(1) == 1 or a.shape[1] <= 1)
        return max(a.stride(0), a.shape[1], 1) if a.shape[0] > 1 else max(a.shape[1], 1)
    assert a.ndim == 2 and (a.strides[1] == a.itemsize or a.shape[1] <= 1)
    return max(a.strides[0] // a.itemsize, a.shape[1], 1) if a.shape[0] > 1 else max(a.shape[1], 1)


def _is_f64(a):
    return "float64" in str(a.dtype)


def _stream(stream):
    if stream is None:
        return None
    return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)


def current_stream_for(*arrays):
    """torch's current stream when any operand is a CUDA tensor, else null."""
    for a in arrays:
        if a is not None and _is_torch(a) and a.is_cuda:
            import torch
            return torch.cuda.current_stream(a.device).cuda_stream
    return None


def gemm(alpha, A, B, beta, Cm, stream=None):
    """Cm = alpha*A@B + beta*Cm in place (fp64 -> pgb200Dgemm, fp32 -> pgb200Sgemm)."""
    M, K = A.shape
    N = B.shape[1]
    assert B.shape[0] == K and tuple(Cm.shape) == (M, N)
    s = _stream(stream) if stream is not None else current_stream_for(A, B, Cm)
    fn = load().pgb200Dgemm if _is_f64(Cm) else load().pgb200Sgemm
    check(fn(s, M, N, K, alpha, _ptr(A), _ld(A), _ptr(B), _ld(B), beta, _ptr(Cm), _ld(Cm)))
    return Cm


def gemm_nt(alpha, A, B, beta, Cm, stream=None):
    """Cm = alpha*A@B^T + beta*Cm in place (A [M,K], B [N,K])."""
    M, K = A.shape
    N = B.shape[0]
    assert B.shape[1] == K and tuple(Cm.shape) == (M, N)
    s = _stream(stream) if stream is not None else current_stream_for(A, B, Cm)
    fn = load().pgb200DgemmNT if _is_f64(Cm) else load().pgb200SgemmNT
    check(fn(s, M, N, K, alpha, _ptr(A), _ld(A), _ptr(B), _ld(B), beta, _ptr(Cm), _ld(Cm)))
    return Cm


def syr2k(alpha, A, B, beta, Cm, stream=None):
    """Lower triangle of Cm = alpha*(A@B^T + B@A^T) + beta*Cm in place."""
    N, K = A.shape
    assert tuple(B.shape) == (N, K) and tuple(Cm.shape) == (N, N)
    s = _stream(stream) if stream is not None else current_stream_for(A, B, Cm)
    fn = load().pgb200Dsyr2k if _is_f64(Cm) else load().pgb200Ssyr2k
    check(fn(s, N, K, alpha, _ptr(A), _ld(A), _ptr(B), _ld(B), beta, _ptr(Cm), _ld(Cm)))
    return Cm


def symm(alpha, A, B, beta, Cm, stream=None):
    """Cm = beta*Cm + alpha*S@B in place, S symmetric with its lower triangle in A."""
    M, N = Cm.shape
    assert tuple(A.shape) == (M, M) and tuple(B.shape) == (M, N)
    s = _stream(stream) if stream is not None else current_stream_for(A, B, Cm)
    fn = load().pgb200Dsymm if _is_f64(Cm) else load().pgb200Ssymm
    check(fn(s, M, N, alpha, _ptr(A), _ld(A), _ptr(B), _ld(B), beta, _ptr(Cm), _ld(Cm)))
    return Cm


def trmm(alpha, A, B, stream=None):
    """B = alpha*(I + L^T)@B in place, L the strict lower triangle of A."""
    M, N = B.shape
    assert tuple(A.shape) == (M, M)
    s = _stream(stream) if stream is not None else current_stream_for(A, B)
    fn = load().pgb200Dtrmm if _is_f64(B) else load().pgb200Strmm
    check(fn(s, M, N, alpha, _ptr(A), _ld(A), _ptr(B), _ld(B)))
    return B


def doitgen(A, C4, sum_=None, stream=None):
    """A[R x P] = A @ C4 in place (float64); `sum_` receives the last row."""
    R, P = A.shape
    assert tuple(C4.shape) == (P, P) and _is_f64(A)
    s = _stream(stream) if stream is not None else current_stream_for(A, C4)
    check(load().pgb200Ddoitgen(s, R, P, _ptr(A), _ld(A), _ptr(C4), _ld(C4),
                                _ptr(sum_) if sum_ is not None else None))
    return A


def syrk(alpha, A, beta, Cm, stream=None, rows=None):
    """Lower triangle of Cm = alpha*A@A^T + beta*Cm in place; `rows=(r0,r1)`
    restricts the update to that row block (fp32 only)."""
    N, K = A.shape
    assert tuple(Cm.shape) == (N, N)
    s = _stream(stream) if stream is not None else current_stream_for(A, Cm)
    if rows is not None:
        assert not _is_f64(Cm)
        check(load().pgb200SsyrkRows(s, N, K, rows[0], rows[1], alpha, _ptr(A), _ld(A), beta,
                                     _ptr(Cm), _ld(Cm)))
        return Cm
    fn = load().pgb200Dsyrk if _is_f64(Cm) else load().pgb200Ssyrk
    check(fn(s, N, K, alpha, _ptr(A), _ld(A), beta, _ptr(Cm), _ld(Cm)))
    return Cm


def syrk_rows(alpha, A, beta, C_block, r0, r1, stream=None):
    """Rows [r0,r1) of the lower-triangular update when only that row block of C
    is resident: `C_block` is the [r1-r0, N] slice, `A` holds rows [0,r1)."""
    K = A.shape[1]
    N = C_block.shape[1]
    assert A.shape[0] >= r1 and C_block.shape[0] == r1 - r0 and not _is_f64(C_block)
    ldc = _ld(C_block)
    # The ABI takes the address of row 0 of C; only rows [r0,r1) are touched.
    base = _ptr(C_block) - r0 * ldc * 4
    s = _stream(stream) if stream is not None else current_stream_for(A, C_block)
    check(load().pgb200SsyrkRows(s, N, K, r0, r1, alpha, _ptr(A), _ld(A), beta, base, ldc))
    return C_block


def gemm_mg(ndev, alpha, A, B, beta, Cm):
    """Cm = alpha*A@B + beta*Cm on `ndev` GPUs from this one process (host arrays
    or tensors of device 0); returns when Cm holds the result."""
    M, K = A.shape
    N = B.shape[1]
    fn = load().pgb200DgemmMg if _is_f64(Cm) else load().pgb200SgemmMg
    check(fn(ndev, M, N, K, alpha, _ptr(A), _ld(A), _ptr(B), _ld(B), beta, _ptr(Cm), _ld(Cm)))
    return Cm


def syrk_mg(ndev, alpha, A, beta, Cm):
    """Lower triangle of Cm = alpha*A@A^T + beta*Cm on `ndev` GPUs (fp32)."""
    N, K = A.shape
    check(load().pgb200SsyrkMg(ndev, N, K, alpha, _ptr(A), _ld(A), beta, _ptr(Cm), _ld(Cm)))
    return Cm


def gemv(trans, alpha, A, x, beta, y, stream=None):
    M, N = A.shape
    s = _stream(stream) if stream is not None else current_stream_for(A, x, y)
    check(load().pgb200Dgemv(s, 1 if trans else 0, M, N, alpha, _ptr(A), _ld(A), _ptr(x), beta,
                             _ptr(y)))
    return y


def gemv_pair(alpha, A, x1, x2, beta, y1, y2, stream=None):
    """y1 = alpha*A@x1 + beta*y1 ; y2 = alpha*A^T@x2 + beta*y2 in one pass over A."""
    M, N = A.shape
    s = _stream(stream) if stream is not None else current_stream_for(A, y1, y2)
    check(load().pgb200DgemvPair(s, M, N, alpha, _ptr(A), _ld(A), _ptr(x1), _ptr(x2), beta,
                                 _ptr(y1), _ptr(y2)))
    return y1, y2


def mvt(A, y1, y2, x1, x2, stream=None):
    """x1 += A@y1 ; x2 += A^T@y2 in one pass over A."""
    N = A.shape[0]
    assert A.shape[1] == N
    s = _stream(stream) if stream is not None else current_stream_for(A, x1, x2)
    check(load().pgb200Dmvt(s, N, _ptr(A), _ld(A), _ptr(y1), _ptr(y2), _ptr(x1), _ptr(x2)))
    return x1, x2


def fill_uniform(t, seed, array_id, lo, hi, row0=0, logical_cols=None, stream=None):
    """Fill a CUDA tensor (1-D or row-major 2-D) with the harness generator."""
    if t.dim() == 1:
        rows, cols, ld = 1, t.shape[0], max(t.shape[0], 1)
    else:
        rows, cols, ld = t.shape[0], t.shape[1], _ld(t)
    assert logical_cols is None or logical_cols == cols
    s = _stream(stream) if stream is not None else current_stream_for(t)
    fn = load().pgb200FillUniformF64 if _is_f64(t) else load().pgb200FillUniformF32
    check(fn(s, _ptr(t), row0, rows, cols, ld, seed, array_id, lo, hi))
    return t


PEAK_DMMA, PEAK_DFMA, PEAK_HBM_READ, PEAK_TF32 = 0, 1, 2, 3


def probe_peak(kind, stream=None):
    """Measured peak of this GPU for `kind` (GFLOP/s or GB/s): a register-only
    tensor/FMA issue loop or a read-only HBM sweep.  Roofline denominators."""
    out = _f64(0.0)
    check(load().pgb200ProbePeak(_stream(stream), kind, C.byref(out)))
    return out.value
