"""Time one libpgb200 entry point on device-resident operands.

    python optime.py --op dsymm --m 4096 --n 4096
    python optime.py --op dtrmm --m 8192 --n 4096 --iters 10

Operands are filled on the device by the library's seeded generator; every
iteration is timed with CUDA events on the launching stream after a write
larger than L2, and one JSON line is printed (median and best time, useful
GFLOP/s for the op's algorithmic flop count, the kernel path taken and the
number of kernels launched per call).
"""
import argparse
import json
import os
import statistics
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

OPS = {
    # name: (dtype, operand shapes as functions of (m, n, k), useful flop)
    "dgemm": ("f64", lambda m, n, k: 2 * m * n * k),
    "sgemm": ("f32", lambda m, n, k: 2 * m * n * k),
    "dsymm": ("f64", lambda m, n, k: 2 * m * m * n),
    "ssymm": ("f32", lambda m, n, k: 2 * m * m * n),
    "dtrmm": ("f64", lambda m, n, k: m * (m - 1) * n),
    "strmm": ("f32", lambda m, n, k: m * (m - 1) * n),
    "dsyrk": ("f64", lambda m, n, k: m * (m + 1) * k),
    "ssyrk": ("f32", lambda m, n, k: m * (m + 1) * k),
    "dsyr2k": ("f64", lambda m, n, k: 2 * m * (m + 1) * k),
    "ssyr2k": ("f32", lambda m, n, k: 2 * m * (m + 1) * k),
    "ddoitgen": ("f64", lambda m, n, k: 2 * m * n * n),
}


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--op", required=True, choices=sorted(OPS))
    ap.add_argument("--m", type=int, default=4096, help="rows (doitgen: NR*NQ)")
    ap.add_argument("--n", type=int, default=4096, help="columns (doitgen: NP)")
    ap.add_argument("--k", type=int, default=4096, help="inner extent (gemm, syrk, syr2k)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--back-to-back", action="store_true",
                    help="time all iterations with one event pair, no L2 flush (launch-bound sizes)")
    ap.add_argument("--no-step-sync", action="store_true",
                    help="pgb200Config.no_step_sync = 1 (two-CTA fp32 kernel without the meeting between rounds)")
    a = ap.parse_args()

    import torch

    import polygeist_b200 as pgb

    if a.no_step_sync:
        pgb.init(no_step_sync=1)

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    dtype, flop = OPS[a.op]
    tdt = torch.float64 if dtype == "f64" else torch.float32
    m, n, k = a.m, a.n, a.k

    def filled(rows, cols, aid):
        t = torch.empty((rows, cols), dtype=tdt, device=dev)
        pgb.fill_uniform(t, 20261125, aid, 0.0, 1.0)
        return t

    kind = a.op[1:]
    if kind == "gemm":
        A, B, Cm = filled(m, k, 1), filled(k, n, 2), filled(m, n, 3)
        call = lambda: pgb.gemm(1.5, A, B, 1.2, Cm)
    elif kind == "symm":
        A, B, Cm = filled(m, m, 1), filled(m, n, 2), filled(m, n, 3)
        call = lambda: pgb.symm(1.5, A, B, 1.2, Cm)
    elif kind == "trmm":
        # alpha = 1/m keeps B bounded over repeated in-place calls
        A, B = filled(m, m, 1), filled(m, n, 2)
        call = lambda: pgb.trmm(1.0 / m, A, B)
    elif kind == "syrk":
        A, Cm = filled(m, k, 1), filled(m, m, 3)
        call = lambda: pgb.syrk(1.5, A, 0.5, Cm)
    elif kind == "syr2k":
        A, B, Cm = filled(m, k, 1), filled(m, k, 2), filled(m, m, 3)
        call = lambda: pgb.syr2k(1.5, A, B, 0.5, Cm)
    else:  # doitgen; C4 scaled so repeated in-place products stay bounded
        A, C4 = filled(m, n, 1), filled(n, n, 2)
        C4.mul_(1.0 / n)
        call = lambda: pgb.doitgen(A, C4)

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # larger than L2
    for _ in range(a.warmup):
        call()
    torch.cuda.synchronize()
    times = []
    launches = 0
    if a.back_to_back:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = pgb.launch_count()
        e0.record()
        for _ in range(a.iters):
            call()
        e1.record()
        e1.synchronize()
        launches = (pgb.launch_count() - l0) // a.iters
        times = [e0.elapsed_time(e1) / a.iters]
    for _ in range(0 if a.back_to_back else a.iters):
        flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = pgb.launch_count()
        e0.record()
        call()
        e1.record()
        e1.synchronize()
        launches = pgb.launch_count() - l0
        times.append(e0.elapsed_time(e1))
    pgb.poll_device_status()
    med, best = statistics.median(times), min(times)
    f = flop(m, n, k)
    print(json.dumps({"op": a.op, "m": m, "n": n, "k": k, "ms_median": round(med, 4),
                      "ms_best": round(best, 4), "gflops_median": round(f / med / 1e6, 1),
                      "gflops_best": round(f / best / 1e6, 1), "useful_flop": f,
                      "path": pgb.last_path(), "launches_per_call": launches, "iters": a.iters,
                      "l2_flush": "none (back to back)" if a.back_to_back
                      else "256 MiB write between iterations"}))


if __name__ == "__main__":
    main()
