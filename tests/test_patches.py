"""CPU checks of the compiler-side deliverables under patches/ (which cannot be
compiled here: no LLVM): the patch applies cleanly to the reference tree when
one is mounted, and the calls it emits have the prototypes include/pgb200.h
declares."""
import os
import re
import shutil
import subprocess

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
PATCH = os.path.join(ROOT, "patches", "raise-affine-to-pgb200.patch")
REF = os.environ.get("PGB200_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))

MLIR_OF_C = {"void *": "!llvm.ptr", "const double *": "!llvm.ptr", "double *": "!llvm.ptr",
             "const float *": "!llvm.ptr", "float *": "!llvm.ptr", "int64_t": "i64",
             "int32_t": "i32", "double": "f64", "float": "f32"}


def _prototype(name):
    text = open(os.path.join(ROOT, "include", "pgb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    m = re.search(r"int32_t\s+" + name + r"\s*\(([^)]*)\)", text)
    assert m, name
    out = []
    for p in m.group(1).split(","):
        p = " ".join(p.split())
        ctype = re.sub(r"\s*\w+$", "", p).strip()       # drop the parameter name
        ctype = ctype.replace(" *", " *")
        out.append(MLIR_OF_C[ctype])
    return out


@pytest.mark.parametrize("name", ["pgb200Dgemm", "pgb200Sgemm", "pgb200Dgemv", "pgb200Dsyrk",
                                  "pgb200Ssyrk", "pgb200Dsyr2k", "pgb200Ssyr2k"])
def test_emitted_calls_match_the_header_prototypes(name):
    """The type lists the pass declares (in the new .cpp inside the patch) and
    the lit test expects are those of the C prototypes."""
    want = _prototype(name)
    lit = open(os.path.join(ROOT, "patches", "test", "raise-affine-to-pgb200.mlir")).read()
    patch = open(PATCH).read()
    if name == "pgb200Dgemm":
        m = re.search(r"func\.func private @pgb200Dgemm\(([^)]*)\) -> i32", lit)
        assert [t.strip() for t in m.group(1).split(",")] == want
    sym = {"f64": "fty", "f32": "fty", "!llvm.ptr": "ptr"}
    if name in ("pgb200Dgemm", "pgb200Sgemm"):
        m = re.search(r"\{ptr, i64, i64, i64, fty, ptr, i64, ptr, i64, fty, ptr, i64\}", patch)
        assert m and [sym.get(t, t) for t in want] == "ptr i64 i64 i64 fty ptr i64 ptr i64 fty ptr i64".split()
    elif name in ("pgb200Dsyr2k", "pgb200Ssyr2k"):
        m = re.search(r"\{ptr, i64, i64, elt, ptr, i64, ptr, i64, elt, ptr, i64\}", patch)
        assert m and [{"f64": "elt", "f32": "elt", "!llvm.ptr": "ptr"}.get(t, t) for t in want] == \
            "ptr i64 i64 elt ptr i64 ptr i64 elt ptr i64".split()
        if name == "pgb200Dsyr2k":
            m = re.search(r"func\.func private @pgb200Dsyr2k\(([^)]*)\) -> i32", lit)
            assert [t.strip() for t in m.group(1).split(",")] == want
    elif name in ("pgb200Dsyrk", "pgb200Ssyrk"):
        m = re.search(r"\{ptr, i64, i64, elt, ptr, i64, elt, ptr, i64\}", patch)
        assert m and [{"f64": "elt", "f32": "elt", "!llvm.ptr": "ptr"}.get(t, t) for t in want] == \
            "ptr i64 i64 elt ptr i64 elt ptr i64".split()
        if name == "pgb200Dsyrk":
            m = re.search(r"func\.func private @pgb200Dsyrk\(([^)]*)\) -> i32", lit)
            assert [t.strip() for t in m.group(1).split(",")] == want
    else:
        m = re.search(r"\{ptr, i32, i64, i64, elt, ptr, i64, ptr, elt, ptr\}", patch)
        assert m and [{"f64": "elt", "!llvm.ptr": "ptr"}.get(t, t) for t in want] == \
            "ptr i32 i64 i64 elt ptr i64 ptr elt ptr".split()


def test_lower_to_target_has_the_reference_signature():
    """pgb200_kernel_gemm takes kernel_gemm's arguments in kernel_gemm's order."""
    text = open(os.path.join(ROOT, "include", "pgb200.h")).read()
    m = re.search(r"int32_t pgb200_kernel_gemm\(([^)]*)\)", text)
    names = [p.split()[-1].lstrip("*") for p in m.group(1).split(",")]
    assert names == ["ni", "nj", "nk", "alpha", "beta", "C", "A", "B"]
    lit = open(os.path.join(ROOT, "patches", "test", "lower_to_pgb200.c")).read()
    assert '#pragma lower_to(kernel_gemm, "func.call @pgb200_kernel_gemm")' in lit


@pytest.mark.skipif(not os.path.isfile(os.path.join(REF, "tools/cgeist/driver.cc")) or
                    shutil.which("patch") is None, reason="no reference tree / patch(1)")
def test_patch_applies_to_the_reference_tree(tmp_path):
    files = sorted(set(re.findall(r"^\+\+\+ b/(\S+)", open(PATCH).read(), flags=re.M)))
    assert "lib/polygeist/Passes/RaiseAffineToPGB200.cpp" in files
    for f in files:
        src = os.path.join(REF, f)
        if os.path.isfile(src):
            os.makedirs(os.path.dirname(tmp_path / f), exist_ok=True)
            shutil.copy(src, tmp_path / f)
    r = subprocess.run(["patch", "-p1", "--batch", "-i", PATCH], cwd=tmp_path, capture_output=True,
                       text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "Hunk" not in r.stdout or "FAILED" not in r.stdout
    drv = open(tmp_path / "tools/cgeist/driver.cc").read()
    assert drv.index("createRaiseSCFToAffinePass()") < drv.index("createRaiseAffineToPGB200Pass()")
