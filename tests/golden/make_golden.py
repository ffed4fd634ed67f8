"""Regenerate the golden text dumps in this directory.

Runs the reference's own verification executables (built by oracle/build.py
from the reference tree with the reference's "%polyverify" flags,
tools/cgeist/Test/lit.cfg:75: -DPOLYBENCH_DUMP_ARRAYS -DMINI_DATASET) and
stores what they print to stderr.  This is the same text the reference's lit
tests diff between clang and cgeist builds (e.g.
tools/cgeist/Test/polybench/linear-algebra/blas/gemm/gemm.c:3-7).

Needs the reference tree; the committed *.dump.txt files are what travels.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..")))

from oracle import build  # noqa: E402


def main():
    out = build.build_ref()
    if out is None:
        sys.exit("reference tree not mounted; nothing regenerated")
    for k in build.KERNELS:
        for t in build.TYPES:
            exe = os.path.join(out, f"{k}_mini_{t}")
            r = subprocess.run([exe], check=True, capture_output=True, text=True)
            path = os.path.join(HERE, f"{k}_mini_{t}.dump.txt")
            with open(path, "w") as f:
                f.write(r.stderr)
            print(path, len(r.stderr), "bytes")


if __name__ == "__main__":
    main()
