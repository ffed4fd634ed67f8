"""Build recipe for the CPU checker.  TEST INFRASTRUCTURE ONLY.

`build_oracle()` compiles this directory's C restatement (pb_oracle.c) into
oracle/libpbo.so.

`build_ref()` compiles the reference's own PolyBench sources *where they lie*
in a mounted reference tree (never copied) into oracle/_ref/:
  libref_<kernel>_<f64|f32>.so   the unmodified kernel_<name> with run-time
                                 array extents (-DPOLYBENCH_USE_C99_PROTO) and
                                 external linkage (-Dstatic=), callable through
                                 ctypes at any size;
  <kernel>_mini_<f64|f32>        the reference's verification executable
                                 (tools/cgeist/Test/lit.cfg:75 "%polyverify":
                                 -DPOLYBENCH_DUMP_ARRAYS -DMINI_DATASET), whose
                                 stderr dump is the golden text under
                                 tests/golden/.
It is a no-op when the reference tree is absent (prebuilt files are used).
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# The reference tree: PGB200_REFERENCE_ROOT, else a checkout named `reference`
# beside this repository.
REF_ROOT = os.environ.get("PGB200_REFERENCE_ROOT",
                          os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
PB = os.path.join(REF_ROOT, "tools/cgeist/Test/polybench")
REF_OUT = os.path.join(HERE, "_ref")

KERNELS = {
    "gemm": "linear-algebra/blas/gemm/gemm.c",
    "2mm": "linear-algebra/kernels/2mm/2mm.c",
    "mvt": "linear-algebra/kernels/mvt/mvt.c",
    "syrk": "linear-algebra/blas/syrk/syrk.c",
    "3mm": "linear-algebra/kernels/3mm/3mm.c",
    "atax": "linear-algebra/kernels/atax/atax.c",
    "bicg": "linear-algebra/kernels/bicg/bicg.c",
    "gesummv": "linear-algebra/blas/gesummv/gesummv.c",
    "syr2k": "linear-algebra/blas/syr2k/syr2k.c",
    "gemver": "linear-algebra/blas/gemver/gemver.c",
    "symm": "linear-algebra/blas/symm/symm.c",
    "trmm": "linear-algebra/blas/trmm/trmm.c",
    "doitgen": "linear-algebra/kernels/doitgen/doitgen.c",
}
TYPES = {"f64": [], "f32": ["-DDATA_TYPE_IS_FLOAT"]}


def _run(cmd):
    subprocess.run(cmd, check=True)


def _newer(dst, srcs):
    if not os.path.exists(dst):
        return False
    t = os.path.getmtime(dst)
    return all(os.path.getmtime(s) <= t for s in srcs)


def build_oracle(force=False):
    srcs = [os.path.join(HERE, f) for f in ("pb_oracle.c", "pb_oracle_impl.h")]
    out = os.path.join(HERE, "libpbo.so")
    if force or not _newer(out, srcs):
        _run(["gcc", "-O2", "-fno-fast-math", "-ffp-contract=off", "-fPIC",
              "-shared", "-o", out, srcs[0]])
    return out


def have_reference():
    return os.path.isfile(os.path.join(PB, "utilities/polybench.c"))


def build_ref(force=False):
    """Compile the reference kernels from the mounted tree.  Returns the
    output directory, or None when there is no reference tree."""
    if not have_reference():
        return None
    os.makedirs(REF_OUT, exist_ok=True)
    util = os.path.join(PB, "utilities")
    pbc = os.path.join(util, "polybench.c")
    pbo = os.path.join(REF_OUT, "polybench_util.o")
    if force or not _newer(pbo, [pbc]):
        _run(["gcc", "-O3", "-fPIC", "-c", "-I", util,
              "-DPOLYBENCH_NO_FLUSH_CACHE", pbc, "-o", pbo])
    for k, rel in KERNELS.items():
        src = os.path.join(PB, rel)
        inc = ["-I", util, "-I", os.path.dirname(src)]
        for t, tdef in TYPES.items():
            lib = os.path.join(REF_OUT, f"libref_{k}_{t}.so")
            if force or not _newer(lib, [src]):
                # x86-64-v3 (AVX2+FMA) rather than -march=native: the file is
                # built on one host and timed on another.
                _run(["gcc", "-O3", "-march=x86-64-v3", "-fPIC", "-shared",
                      "-DPOLYBENCH_USE_C99_PROTO", "-Dstatic=",
                      "-Dmain=pb_unused_main", *tdef, *inc, src, pbo,
                      "-lm", "-o", lib])
            exe = os.path.join(REF_OUT, f"{k}_mini_{t}")
            if force or not _newer(exe, [src]):
                _run(["gcc", "-O3", *tdef, *inc, "-DPOLYBENCH_DUMP_ARRAYS",
                      "-DPOLYBENCH_NO_FLUSH_CACHE", "-DMINI_DATASET", src, pbc,
                      "-lm", "-o", exe])
    return REF_OUT


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
