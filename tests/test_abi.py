"""CPU tests of the drop-in boundary: the shared library loads, exports every
symbol include/pgb200.h declares, and fails loudly (never computes on the CPU)
when there is no GPU."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import polygeist_b200 as pgb

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "pgb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pgb200\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_typed():
    lib = pgb.load()
    names = _declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in pgb200.h but not exported"
        assert n in pgb.SIGNATURES, f"{n} has no ctypes signature"
    assert set(pgb.SIGNATURES) == set(names)


def test_version_and_error_string():
    lib = pgb.load()
    assert lib.pgb200Version() >= 100
    assert isinstance(lib.pgb200GetLastErrorString(), bytes)


def _no_gpu():
    import torch
    return not torch.cuda.is_available()


@pytest.mark.skipif(not _no_gpu(), reason="only meaningful without a GPU")
def test_no_cpu_fallback_without_gpu():
    """Without a device the compute entry points return an error status and
    leave the output untouched - there is no silent host path."""
    lib = pgb.load()
    A = np.ones((4, 4))
    B = np.ones((4, 4))
    Cm = np.full((4, 4), 3.0)
    st = lib.pgb200Dgemm(None, 4, 4, 4, 1.0, A.ctypes.data, 4, B.ctypes.data, 4, 0.0,
                         Cm.ctypes.data, 4)
    assert st in (pgb.ERR_CUDA, pgb.ERR_UNSUPPORTED)
    assert np.all(Cm == 3.0)
    assert lib.pgb200GetLastErrorString() != b""
    with pytest.raises(pgb.PGB200Error):
        from polygeist_b200 import polybench
        polybench.kernel_gemm(4, 4, 4, 1.0, 0.0, Cm, A, B)


def test_polybench_mirror_rejects_wrong_extents():
    from polygeist_b200 import polybench
    with pytest.raises(ValueError):
        polybench.kernel_gemm(4, 4, 4, 1.0, 0.0, np.zeros((4, 5)), np.zeros((4, 4)), np.zeros((4, 4)))
    with pytest.raises(ValueError):
        polybench.kernel_mvt(4, np.zeros(4), np.zeros(4), np.zeros(4), np.zeros(4),
                             np.zeros((4, 4), dtype=np.float32))
    with pytest.raises(ValueError):   # A of symm is m x m
        polybench.kernel_symm(4, 6, 1.5, 1.2, np.zeros((4, 6)), np.zeros((4, 6)), np.zeros((4, 6)))
    with pytest.raises(ValueError):   # B of trmm is m x n, passed transposed
        polybench.kernel_trmm(4, 6, 1.5, np.zeros((4, 4)), np.zeros((6, 4)))
    with pytest.raises(ValueError):   # a strided view is not the C array
        polybench.kernel_trmm(4, 6, 1.5, np.zeros((4, 4)), np.zeros((4, 12))[:, ::2])
    with pytest.raises(ValueError):   # doitgen: A is nr x nq x np
        polybench.kernel_doitgen(2, 3, 4, np.zeros((6, 4)), np.zeros((4, 4)), np.zeros(4))


def build_c_caller(tmp_path):
    """Compile tests/c_harness/polybench_caller.c as strict C99 against the
    public header and link it with the in-tree library."""
    import subprocess
    here = os.path.dirname(os.path.abspath(__file__))
    root = os.path.dirname(here)
    libdir = os.path.dirname(pgb.LIB_PATH)
    pgb.load()  # builds the library when absent
    exe = str(tmp_path / "polybench_caller")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-O1",
                    "-I", os.path.join(root, "include"),
                    os.path.join(here, "c_harness", "polybench_caller.c"), "-o", exe,
                    "-L", libdir, "-lpgb200", "-lm", f"-Wl,-rpath,{libdir}"], check=True)
    return exe


def test_header_is_c99_and_a_c_program_links(tmp_path):
    import subprocess
    exe = build_c_caller(tmp_path)
    out = subprocess.run([exe], check=True, capture_output=True, text=True).stdout
    assert "libpgb200 version" in out


def test_longest_first_tile_schedule():
    """The host-built schedule of the triangular products (an internal C++
    function, reached through its exported symbol): every tile exactly once,
    loads within one tile of each other, oversize problems refused."""
    lib = pgb.load()
    fn = _internal(lib, "build_lpt_schedule")
    fn.restype = C.c_bool
    fn.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.c_void_p]
    MAX_TILES, MAX_WORKERS = 1408, 160

    class Sched(C.Structure):
        _fields_ = [("off", C.c_uint16 * (MAX_WORKERS + 1)), ("idx", C.c_uint16 * MAX_TILES)]

    rng = np.random.default_rng(3)
    for tiles, workers in ((1024, 148), (256, 74), (149, 148), (7, 3), (0, 5)):
        cost = np.sort(rng.integers(1, 260, tiles).astype(np.int64))[::-1].copy()
        s = Sched()
        assert fn(cost.ctypes.data, tiles, workers, C.addressof(s))
        off = np.array(s.off[: workers + 1], dtype=np.int64)
        assert off[0] == 0 and off[-1] == tiles and np.all(np.diff(off) >= 0)
        idx = np.array(s.idx[:tiles], dtype=np.int64)
        assert sorted(idx.tolist()) == list(range(tiles))
        loads = np.array([cost[idx[off[w]:off[w + 1]]].sum() for w in range(workers)])
        if tiles >= workers:
            assert loads.max() - loads.min() <= cost.max()
            # within a worker the tiles come longest first
            for w in range(workers):
                mine = cost[idx[off[w]:off[w + 1]]]
                assert np.all(np.diff(mine) <= 0)
    big = np.ones(MAX_TILES + 1, dtype=np.int64)
    assert not fn(big.ctypes.data, MAX_TILES + 1, 148, C.addressof(Sched()))
    assert not fn(big.ctypes.data, 10, MAX_WORKERS + 1, C.addressof(Sched()))


def _internal(lib, fragment):
    """An internal C++ function of the library, by a fragment of its mangled name."""
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", pgb.LIB_PATH], check=True,
                         capture_output=True, text=True).stdout
    names = [ln.split()[-1] for ln in out.splitlines() if fragment in ln]
    assert len(names) == 1, names
    return getattr(lib, names[0])


@pytest.mark.parametrize("M,N,bm,bn,lower,row0", [
    (1024, 1024, 128, 256, 0, 0), (1000, 1100, 128, 64, 0, 0), (4096, 2048, 256, 256, 0, 0),
    (130, 70, 128, 256, 0, 0),                       # fewer tile rows than a band
    (2048, 2048, 128, 256, 1, 0), (1200, 1200, 128, 64, 1, 0), (2048, 2048, 256, 256, 1, 0),
    (768, 1408, 128, 256, 1, 640), (200, 640, 128, 64, 1, 440), (768, 1408, 256, 256, 1, 640),
    (2100, 2100, 128, 256, 1, 0),                    # more than one band of 16 tile rows
])
def test_fp32_tile_walk_covers_every_tile_once(M, N, bm, bn, lower, row0):
    """The band-ordered walk of the fp32 kernels: every tile that holds an
    element with j <= i + row0 (or every tile, for a full product) is visited
    exactly once, and the host-side count agrees with the walk."""
    lib = pgb.load()
    fn = _internal(lib, "enumerate_tiles_for_test")
    fn.restype = C.c_int64
    fn.argtypes = [C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_void_p,
                   C.c_void_p, C.c_int64]
    cap = 1 << 16
    tm = np.zeros(cap, dtype=np.int64)
    tn = np.zeros(cap, dtype=np.int64)
    n = fn(M, N, bm, bn, lower, row0, tm.ctypes.data, tn.ctypes.data, cap)
    assert n >= 0
    got = list(zip(tm[:n].tolist(), tn[:n].tolist()))
    want = set()
    for r in range(-(-M // bm)):
        for c in range(-(-N // bn)):
            # lower: the tile row's last row (r*bm + bm - 1, absolute + row0) reaches column c*bn
            if not lower or c * bn <= r * bm + bm - 1 + row0:
                want.add((r, c))
    assert len(got) == len(set(got)), "a tile is visited twice"
    assert set(got) == want


@pytest.mark.parametrize("tiles_m,tiles_n,lower", [(32, 32, 0), (7, 3, 0), (1, 9, 0), (19, 5, 0),
                                                   (1, 1, 1), (10, 10, 1), (64, 64, 1), (181, 181, 1)])
def test_fp64_tile_map_is_a_bijection(tiles_m, tiles_n, lower):
    """Linear tile index -> (row, column) of the fp64 kernel: groups of 8 tile
    rows for a full product, the packed lower triangle (square-root inverse)
    for the triangular update."""
    lib = pgb.load()
    fn = _internal(lib, "enumerate_dmma_tiles_for_test")
    fn.restype = C.c_int64
    fn.argtypes = [C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_int64]
    cap = 1 << 16
    tm = np.zeros(cap, dtype=np.int64)
    tn = np.zeros(cap, dtype=np.int64)
    n = fn(tiles_m, tiles_n, lower, tm.ctypes.data, tn.ctypes.data, cap)
    got = list(zip(tm[:n].tolist(), tn[:n].tolist()))
    if lower:
        want = {(r, c) for r in range(tiles_m) for c in range(r + 1)}
    else:
        want = {(r, c) for r in range(tiles_m) for c in range(tiles_n)}
    assert n == len(want) and len(set(got)) == n and set(got) == want
